// Decode-shaped mat-mul (few activation rows): HBM-bound streaming kernels.
//
// One CTA owns one 32-row tile of the weight matrix; lane r of every warp owns
// row r, the warps split the 256-element groups of K between them.  Each lane
// reads its row's bytes of a group with 16-byte loads that are contiguous
// across the warp (512 B per load instruction), does the integer block dots
// with dp4a against the Q8 activations (staged per warp in shared memory and
// read as broadcasts), and leaves the exact int32 partials in shared memory.
// After one barrier the f32 accumulation chains are run in ascending K order,
// exactly as the CPU route does, so the result is bit-identical to it:
//   Q4_K 8x8 gemv   crates/ggml/src/repack.rs:1638-1688 (one fma per super-block
//                   for the scale term and one for the min term, out = acc - accmin)
#include <cstdlib>

#include "common.cuh"
#include "act_quant.cuh"
#include "fa_math.cuh"
#include "gemv_types.cuh"

namespace b200 {

constexpr int GEMV_MAX_WARPS = 16;

// MUL_MAT_ID: blockIdx.y walks the (token, slot) pairs; each pair picks its expert's weights, its
// activation row (slot % ne11 of its token) and its output row (crates/ggml/src/compute.rs:2104-2130).
// counts/min_count/max_count let two launches with different chains split the pairs by how many rows
// were routed to the pair's expert (the tiled chain from 8 rows on, the row dot below).
struct PairMap {
    const int32_t *ids;      // [n_tok][n_ids], null for plain MUL_MAT
    int n_ids, ne11, n_expert;
    int64_t expert_bytes;
    const int *counts;       // rows routed to each expert, or null
    int min_count, max_count;
    // plain MUL_MAT over several matrices that read the same activation row (k, v, q of a layer; gate and up of
    // an FFN) in one launch: blockIdx.x walks the row tiles of all of them, segment 0 being the kernel's own
    // tiles / dst / n arguments and segments 1.. the ones below
    int seg_count;           // 0 or 1: a single matrix
    int seg_end[2];          // first tile of segment 1 and of segment 2 (INT_MAX: no segment 2)
    int seg_total;           // tiles of all segments
    // K split (one activation row, few row tiles): blockIdx.z walks ksplit ranges of super-blocks; every CTA leaves
    // its integer partials in kx[tile][nb][32], and the last one to arrive at kcount[tile] runs the f32 chain over
    // all of K in order, so the result does not depend on the split
    int ksplit;              // 0 or 1: no split
    int4 *kx;
    int *kcount;
    const uint8_t *seg_tiles[2];
    float *seg_dst[2];
    int64_t seg_n[2];
};

__device__ __forceinline__ bool apply_pair(const PairMap &pm, const uint8_t *&tiles, ActView &acts, float *&dst,
                                           int64_t lddst) {
    if (!pm.ids) return true;
    const int64_t pair = blockIdx.y;
    const int e = pm.ids[pair];
    if (e < 0 || e >= pm.n_expert) return false;
    if (pm.counts) {
        const int c = pm.counts[e];
        if (c < pm.min_count || c > pm.max_count) return false;
    }
    const int64_t tok = pair / pm.n_ids, slot = pair % pm.n_ids;
    const int64_t arow = tok * pm.ne11 + slot % pm.ne11;
    tiles += (int64_t)e * pm.expert_bytes;
    acts.qs += arow * acts.k;
    if (acts.d) acts.d += arow * (acts.k / 256);
    if (acts.bsums) acts.bsums += arow * (acts.k / 16);
    if (acts.dh) acts.dh += arow * (acts.k / 32);
    dst += pair * lddst;
    return true;
}

// ---------------------------------------------------------------------------
// Q4_K, route REPACK/gemv.  NCOL activation rows share one pass over the weights.
// Shared memory: per warp staging of one activation group per column, and the
// exchange array xch[col][group][row] = {iacc, imin, d|dmin<<16}.
// ---------------------------------------------------------------------------
struct Q4KStage {
    uint4 q[16];   // 256 activation quants of one group
    int bp[8];     // bsums[2j] + bsums[2j+1]
};

// MODE selects the f32 chain of the mirrored CPU route:
//   0  8x8 gemv  (repack.rs:1638-1688): one fma per super-block and term, out = acc - accmin
//   1  8x8 gemm  (repack.rs:1692-1768): one fma per (super-block, sub-block pair) and term
//   2  tiled     (tiled.rs:823-838):    r = d*f32(s1); r = fma(-dmin, f32(s2), r); out = fma(r, d_x, out)
// PF: a warp that walks several groups of K (long rows, few row tiles: one CTA per SM anyway) issues the loads of
// its next group before it computes the current one; costs 36 registers, so only such shapes are launched with it.
template <int NCOL, int MODE, bool PF = false>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_q4_K_kernel(const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, PairMap pm) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger();
    if (pm.ids) pdl_wait();   // the expert ids come from a previous kernel
    if (!apply_pair(pm, tiles, acts, dst, lddst)) return;
    int tile = blockIdx.x;
    if (pm.seg_count > 1) {   // constant indices only: the segment table stays in the parameter bank
        if (tile >= pm.seg_end[1]) {
            tile -= pm.seg_end[1];
            tiles = pm.seg_tiles[1];
            dst = pm.seg_dst[1];
            n = pm.seg_n[1];
        } else if (tile >= pm.seg_end[0]) {
            tile -= pm.seg_end[0];
            tiles = pm.seg_tiles[0];
            dst = pm.seg_dst[0];
            n = pm.seg_n[0];
        }
    }
    bool waited = pm.ids != nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    Q4KStage *stage = (Q4KStage *)smem + warp * NCOL;
    constexpr int XW = MODE == 1 ? 3 : 1;                           // int4 words per (col, group, row)
    int4 *xch = (int4 *)(smem + sizeof(Q4KStage) * nwarps * NCOL);  // [NCOL][nb][XW][32]
    const uint8_t *base = tiles + tile * (int64_t)nb * 4608;
    int b_first = 0, b_last = nb;
    if (pm.ksplit > 1) {
        const int per = (nb + pm.ksplit - 1) / pm.ksplit;
        b_first = (int)blockIdx.z * per;
        b_last = b_first + per < nb ? b_first + per : nb;
    }
    int4 *gx = pm.ksplit > 1 ? pm.kx + (int64_t)tile * nb * 32 : nullptr;

    uint4 h_n = make_uint4(0, 0, 0, 0), q_n[8];
    if (PF && b_first + warp < b_last) {
        const uint8_t *chunk = base + (int64_t)(b_first + warp) * 4608;
        h_n = ld_stream16(chunk + lane * 16);
#pragma unroll
        for (int c = 0; c < 8; c++) q_n[c] = ld_stream16(chunk + 512 + c * 512 + lane * 16);
    }
    for (int b = b_first + warp; b < b_last; b += nwarps) {
        const uint8_t *chunk = base + (int64_t)b * 4608;
        uint4 h, q[8];
        if (PF) {
            h = h_n;
#pragma unroll
            for (int c = 0; c < 8; c++) q[c] = q_n[c];
            if (b + nwarps < b_last) {
                const uint8_t *next = chunk + (int64_t)nwarps * 4608;
                h_n = ld_stream16(next + lane * 16);
#pragma unroll
                for (int c = 0; c < 8; c++) q_n[c] = ld_stream16(next + 512 + c * 512 + lane * 16);
            }
        } else {
            h = ld_stream16(chunk + lane * 16);
#pragma unroll
            for (int c = 0; c < 8; c++) q[c] = ld_stream16(chunk + 512 + c * 512 + lane * 16);
        }
        // the weight loads above are in flight; the activations are the previous kernel's output
        if (!waited) { pdl_wait(); waited = true; }
        // stage this group's activations for every column
#pragma unroll
        for (int col = 0; col < NCOL; col++) {
            if (lane < 16) {
                stage[col].q[lane] = *(const uint4 *)(acts.qs + (int64_t)col * acts.k + (int64_t)b * 256 + lane * 16);
            } else if (lane < 24) {
                const int j = lane - 16;
                const short2 s2 = *(const short2 *)(acts.bsums + (int64_t)col * (acts.k / 16) + (int64_t)b * 16 + 2 * j);
                stage[col].bp[j] = (int)s2.x + (int)s2.y;
            }
        }
        __syncwarp();
        // 6-bit scales and mins: crates/ggml/src/quants.rs:421-429 (get_scale_min_k4)
        const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
        const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu;                                         // scales 0..3
        const uint32_t mn_lo4 = u1 & 0x3f3f3f3fu;                                         // mins   0..3
        const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);    // scales 4..7
        const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);  // mins 4..7
#pragma unroll
        for (int col = 0; col < NCOL; col++) {
            int iacc = 0;
            int ig[4], mg[4];
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int dlo = 0, dhi = 0;
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint4 w = q[2 * g + hh];
                    const uint4 alo = stage[col].q[4 * g + hh];      // elements 64g + 16hh ..
                    const uint4 ahi = stage[col].q[4 * g + 2 + hh];  // elements 64g + 32 + 16hh ..
                    dlo = __dp4a((int)(w.x & 0x0f0f0f0fu), (int)alo.x, dlo);
                    dlo = __dp4a((int)(w.y & 0x0f0f0f0fu), (int)alo.y, dlo);
                    dlo = __dp4a((int)(w.z & 0x0f0f0f0fu), (int)alo.z, dlo);
                    dlo = __dp4a((int)(w.w & 0x0f0f0f0fu), (int)alo.w, dlo);
                    dhi = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, dhi);
                    dhi = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, dhi);
                    dhi = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, dhi);
                    dhi = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, dhi);
                }
                const uint32_t s4 = g < 2 ? sc_lo4 : sc_hi4;
                const int s_lo = (s4 >> (16 * (g & 1))) & 0xff;
                const int s_hi = (s4 >> (16 * (g & 1) + 8)) & 0xff;
                ig[g] = dlo * s_lo + dhi * s_hi;
                iacc += ig[g];
            }
            int imin = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t m4 = j < 4 ? mn_lo4 : mn_hi4;
                const int term = (int)((m4 >> (8 * (j & 3))) & 0xff) * stage[col].bp[j];
                imin += term;
                if (j & 1) mg[j >> 1] += term; else mg[j >> 1] = term;
            }
            int4 *xe = xch + ((int64_t)col * nb + b) * XW * 32 + lane;
            if (MODE == 1) {
                xe[0] = make_int4(ig[0], ig[1], ig[2], ig[3]);
                xe[32] = make_int4(mg[0], mg[1], mg[2], mg[3]);
                xe[64] = make_int4((int)h.x, 0, 0, 0);
            } else if (gx) {
                gx[(int64_t)b * 32 + lane] = make_int4(iacc, imin, (int)h.x, 0);
            } else {
                xe[0] = make_int4(iacc, imin, (int)h.x, 0);
            }
        }
        __syncwarp();
    }
    if (!waited) pdl_wait();
    if (gx) {
        // the last CTA of the tile to get here has every range's partials in front of it
        __shared__ int is_last;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) is_last = atomicAdd(&pm.kcount[tile], 1) == pm.ksplit - 1;
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        if (threadIdx.x == 0) pm.kcount[tile] = 0;   // ready for the next launch
    }
    __syncthreads();
    // accumulation chains, ascending K: threads (col, row)
    for (int t = threadIdx.x; t < NCOL * 32; t += blockDim.x) {
        const int col = t >> 5, r = t & 31;
        const float *dx = acts.d + (int64_t)col * nb;
        float sumf = 0.0f, summin = 0.0f;
#pragma unroll 4
        for (int b = 0; b < nb; b++) {
            const int4 *xe = xch + ((int64_t)col * nb + b) * XW * 32 + r;
            const float da = dx[b];
            if (MODE == 1) {
                const int4 vi = xe[0], vm = xe[32];
                const uint32_t hd = (uint32_t)xe[64].x;
                const float sd = __fmul_rn(f16_bits_to_f32((uint16_t)(hd & 0xffffu)), da);
                const float sm = __fmul_rn(f16_bits_to_f32((uint16_t)(hd >> 16)), da);
                sumf = __fmaf_rn((float)vi.x, sd, sumf); summin = __fmaf_rn((float)vm.x, sm, summin);
                sumf = __fmaf_rn((float)vi.y, sd, sumf); summin = __fmaf_rn((float)vm.y, sm, summin);
                sumf = __fmaf_rn((float)vi.z, sd, sumf); summin = __fmaf_rn((float)vm.z, sm, summin);
                sumf = __fmaf_rn((float)vi.w, sd, sumf); summin = __fmaf_rn((float)vm.w, sm, summin);
            } else {
                const int4 v = gx ? __ldcg(gx + (int64_t)b * 32 + r) : xe[0];
                const float d = f16_bits_to_f32((uint16_t)((uint32_t)v.z & 0xffffu));
                const float dmin = f16_bits_to_f32((uint16_t)((uint32_t)v.z >> 16));
                if (MODE == 0) {
                    sumf = __fmaf_rn((float)v.x, __fmul_rn(d, da), sumf);
                    summin = __fmaf_rn((float)v.y, __fmul_rn(dmin, da), summin);
                } else {
                    float rr = __fmul_rn(d, (float)v.x);
                    rr = __fmaf_rn(-dmin, (float)v.y, rr);
                    sumf = __fmaf_rn(rr, da, sumf);
                }
            }
        }
        const int64_t row = (int64_t)tile * TILE_ROWS + r;
        if (row < n) {
            const float v = MODE == 2 ? sumf : __fsub_rn(sumf, summin);
            dst[(int64_t)col * lddst + row] = v;
            if (acts.sum && col == 0) acts.sum[row] = __fadd_rn(v, acts.addend[row]);
        }
    }
}

// ---------------------------------------------------------------------------
// Q4_K, 8x8 gemv chain, ONE activation row: the decode kernel.  The arithmetic of gemv_q4_K_kernel<1, 0>, plus an
// activation prologue: the f32 op that feeds the mat-mul in a decoder layer and the Q8_K quantization of its result
// run inside the mat-mul's CTAs instead of in a kernel of their own (at one token each of those kernels is a few
// microseconds of launch latency for a few KB of work):
//   ACT_PRO_NONE   the activations arrive quantized (ActView)
//   ACT_PRO_PLAIN  quantize x                                         (attention output -> attn_output)
//   ACT_PRO_NORM   quantize (x * rms_scale(x)) * w                    (RMS_NORM + MUL -> q/k/v, gate/up)
//   ACT_PRO_SILU   quantize silu(x) * w                               (SILU + MUL -> ffn_down)
// Every CTA redoes the prologue for the groups of K its warps walk (the row is a few KB and sits in L2); a warp
// quantizes the 256-element block it is about to multiply, with the value rules of quantize_row_q8_K
// (crates/ggml/src/quants.rs:615-654), so the integers that meet the weights are the ones the separate kernels
// would have produced.  The CTA of row tile 0 also writes the prologue's node outputs (norm, weighted norm / silu,
// gated product) and the quantized row, for whatever else reads them.  For ACT_PRO_NORM the CTA first sums the
// row's squares in f64 (crates/ggml/src/compute.rs:2634-2683), while its first weight loads are in flight.
// blockIdx.x walks the row tiles of up to three matrices (PairMap segments), blockIdx.y the (token, slot) pairs of a
// MUL_MAT_ID.  PF: a warp that walks several groups issues the loads of its next group before the current one's
// arithmetic.
// ---------------------------------------------------------------------------
template <bool PF, int PRO>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_q4_K_row_kernel(const uint8_t *tiles, ActView acts, float *dst, int64_t n, int nb, PairMap pm, ActPrologue pro) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger();
    if (pm.ids) pdl_wait();   // the expert ids come from a previous kernel
    if (!apply_pair(pm, tiles, acts, dst, n)) return;
    int tile = blockIdx.x;
    const bool writer = PRO != ACT_PRO_NONE && blockIdx.x == 0 && blockIdx.y == 0;   // materializes the prologue's outputs
    if (pm.seg_count > 1) {   // constant indices only: the segment table stays in the parameter bank
        if (tile >= pm.seg_end[1]) {
            tile -= pm.seg_end[1];
            tiles = pm.seg_tiles[1];
            dst = pm.seg_dst[1];
            n = pm.seg_n[1];
        } else if (tile >= pm.seg_end[0]) {
            tile -= pm.seg_end[0];
            tiles = pm.seg_tiles[0];
            dst = pm.seg_dst[0];
            n = pm.seg_n[0];
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    Q4KStage *stage = (Q4KStage *)smem + warp;
    int4 *xch = (int4 *)(smem + sizeof(Q4KStage) * nwarps);   // [nb][32]
    float *dx_s = (float *)(xch + (size_t)nb * 32);           // [nb] activation block scales
    __shared__ double sq_part[GEMV_MAX_WARPS];
    const uint8_t *base = tiles + tile * (int64_t)nb * 4608;

    uint4 h_n = make_uint4(0, 0, 0, 0), q_n[8];
    if (warp < nb) {
        const uint8_t *chunk = base + (int64_t)warp * 4608;
        h_n = ld_stream16(chunk + lane * 16);
#pragma unroll
        for (int c = 0; c < 8; c++) q_n[c] = ld_stream16(chunk + 512 + c * 512 + lane * 16);
    }
    if (!pm.ids) pdl_wait();   // everything below reads what earlier kernels wrote
    float rms_scale = 1.0f;
    if (PRO == ACT_PRO_NORM) {
        double sum = 0.0;
        for (int b = warp; b < nb; b += nwarps) {
            const float4 a0 = *(const float4 *)(pro.x + (int64_t)b * 256 + 8 * lane), a1 = *(const float4 *)(pro.x + (int64_t)b * 256 + 8 * lane + 4);
            sum += (double)__fmul_rn(a0.x, a0.x); sum += (double)__fmul_rn(a0.y, a0.y);
            sum += (double)__fmul_rn(a0.z, a0.z); sum += (double)__fmul_rn(a0.w, a0.w);
            sum += (double)__fmul_rn(a1.x, a1.x); sum += (double)__fmul_rn(a1.y, a1.y);
            sum += (double)__fmul_rn(a1.z, a1.z); sum += (double)__fmul_rn(a1.w, a1.w);
        }
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) sq_part[warp] = sum;
        __syncthreads();
        double total = 0.0;
        for (int i = 0; i < nwarps; i++) total += sq_part[i];
        const float mean = __double2float_rn(total / (double)(nb * 256));
        rms_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, pro.eps)));
    }

    for (int b = warp; b < nb; b += nwarps) {
        uint4 h = h_n, q[8];
#pragma unroll
        for (int c = 0; c < 8; c++) q[c] = q_n[c];
        if (PF && b + nwarps < nb) {
            const uint8_t *next = base + (int64_t)(b + nwarps) * 4608;
            h_n = ld_stream16(next + lane * 16);
#pragma unroll
            for (int c = 0; c < 8; c++) q_n[c] = ld_stream16(next + 512 + c * 512 + lane * 16);
        }
        // this group's activations into the warp's stage
        if (PRO == ACT_PRO_NONE) {
            if (lane < 16) {
                stage->q[lane] = *(const uint4 *)(acts.qs + (int64_t)b * 256 + lane * 16);
            } else if (lane < 24) {
                const int j = lane - 16;
                const short2 s2 = *(const short2 *)(acts.bsums + (int64_t)b * 16 + 2 * j);
                stage->bp[j] = (int)s2.x + (int)s2.y;
            } else if (lane == 24) {
                dx_s[b] = acts.d[b];
            }
        } else {
            const int64_t e0 = (int64_t)b * 256 + 8 * lane;
            float v[8];
            {
                const float4 a0 = *(const float4 *)(pro.x + e0), a1 = *(const float4 *)(pro.x + e0 + 4);
                v[0] = a0.x; v[1] = a0.y; v[2] = a0.z; v[3] = a0.w; v[4] = a1.x; v[5] = a1.y; v[6] = a1.z; v[7] = a1.w;
            }
            if (PRO == ACT_PRO_NORM) {
                const float4 w0 = *(const float4 *)(pro.w + e0), w1 = *(const float4 *)(pro.w + e0 + 4);
                const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                float nv[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    nv[j] = __fmul_rn(v[j], rms_scale);
                    v[j] = __fmul_rn(nv[j], ws[j]);
                }
                if (writer) {
                    if (pro.y) {
                        *(float4 *)(pro.y + e0) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                        *(float4 *)(pro.y + e0 + 4) = make_float4(nv[4], nv[5], nv[6], nv[7]);
                    }
                    *(float4 *)(pro.y_mul + e0) = make_float4(v[0], v[1], v[2], v[3]);
                    *(float4 *)(pro.y_mul + e0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
            } else if (PRO == ACT_PRO_SILU) {
                const float4 g0 = *(const float4 *)(pro.w + e0), g1 = *(const float4 *)(pro.w + e0 + 4);
                const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                float sv[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float e = (int)(e0 + j) < pro.wide_end ? v_expf(__fsub_rn(0.0f, v[j])) : libm_expf(-v[j]);
                    sv[j] = __fdiv_rn(v[j], __fadd_rn(1.0f, e));
                    v[j] = __fmul_rn(sv[j], gs[j]);
                }
                if (writer) {
                    if (pro.y) {
                        *(float4 *)(pro.y + e0) = make_float4(sv[0], sv[1], sv[2], sv[3]);
                        *(float4 *)(pro.y + e0 + 4) = make_float4(sv[4], sv[5], sv[6], sv[7]);
                    }
                    *(float4 *)(pro.y_mul + e0) = make_float4(v[0], v[1], v[2], v[3]);
                    *(float4 *)(pro.y_mul + e0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
            }
            // quantize_row_q8_K on the block the warp holds (lane l: elements 8 l .. 8 l + 7)
            uint2 packed;
            float d;
            int s8;
            q8_K_block_regs(v, &packed, &d, &s8);
            *(uint2 *)((unsigned char *)stage->q + 8 * lane) = packed;
            int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);        // a 16-element sum is two lanes
            const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);  // bsums[2j] + bsums[2j+1] is four lanes
            if ((lane & 3) == 0) stage->bp[lane >> 2] = s32;
            if (lane == 0) dx_s[b] = d;
            if (writer && pro.act_out.qs) {
                *(uint2 *)(pro.act_out.qs + e0) = packed;
                if ((lane & 1) == 0) pro.act_out.bsums[(int64_t)b * 16 + (lane >> 1)] = (int16_t)s16;
                if (lane == 0) pro.act_out.d[b] = d;
            }
        }
        __syncwarp();
        // 6-bit scales and mins: crates/ggml/src/quants.rs:421-429 (get_scale_min_k4)
        const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
        const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu, mn_lo4 = u1 & 0x3f3f3f3fu;
        const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
        const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
        int iacc = 0;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            int dlo = 0, dhi = 0;
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const uint4 w = q[2 * g + hh];
                const uint4 alo = stage->q[4 * g + hh], ahi = stage->q[4 * g + 2 + hh];
                dlo = __dp4a((int)(w.x & 0x0f0f0f0fu), (int)alo.x, dlo);
                dlo = __dp4a((int)(w.y & 0x0f0f0f0fu), (int)alo.y, dlo);
                dlo = __dp4a((int)(w.z & 0x0f0f0f0fu), (int)alo.z, dlo);
                dlo = __dp4a((int)(w.w & 0x0f0f0f0fu), (int)alo.w, dlo);
                dhi = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, dhi);
                dhi = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, dhi);
                dhi = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, dhi);
                dhi = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, dhi);
            }
            const uint32_t s4 = g < 2 ? sc_lo4 : sc_hi4;
            iacc += dlo * (int)((s4 >> (16 * (g & 1))) & 0xff) + dhi * (int)((s4 >> (16 * (g & 1) + 8)) & 0xff);
        }
        int imin = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t m4 = j < 4 ? mn_lo4 : mn_hi4;
            imin += (int)((m4 >> (8 * (j & 3))) & 0xff) * stage->bp[j];
        }
        xch[b * 32 + lane] = make_int4(iacc, imin, (int)h.x, 0);
        __syncwarp();
        if (!PF && b + nwarps < nb) {   // without the prefetch the next group is loaded only now
            const uint8_t *next = base + (int64_t)(b + nwarps) * 4608;
            h_n = ld_stream16(next + lane * 16);
#pragma unroll
            for (int c = 0; c < 8; c++) q_n[c] = ld_stream16(next + 512 + c * 512 + lane * 16);
        }
    }
    __syncthreads();
    // accumulation chain, ascending K: one warp, lane = row
    if (warp == 0) {
        float sumf = 0.0f, summin = 0.0f;
#pragma unroll 4
        for (int bb = 0; bb < nb; bb++) {
            const int4 v = xch[bb * 32 + lane];
            const float d = f16_bits_to_f32((uint16_t)((uint32_t)v.z & 0xffffu));
            const float dmin = f16_bits_to_f32((uint16_t)((uint32_t)v.z >> 16));
            const float da = dx_s[bb];
            sumf = __fmaf_rn((float)v.x, __fmul_rn(d, da), sumf);
            summin = __fmaf_rn((float)v.y, __fmul_rn(dmin, da), summin);
        }
        const int64_t row = (int64_t)tile * TILE_ROWS + lane;
        if (row < n) {
            const float v = __fsub_rn(sumf, summin);
            dst[row] = v;
            if (acts.sum) acts.sum[row] = __fadd_rn(v, acts.addend[row]);
        }
    }
}

static int pick_warps(int nb) {
    // the largest warp count <= 16 that divides the group count keeps every warp equally loaded
    for (int w = GEMV_MAX_WARPS; w >= 8; w--)
        if (nb % w == 0) return w;
    return nb < GEMV_MAX_WARPS ? (nb < 1 ? 1 : nb) : GEMV_MAX_WARPS;
}

template <int NCOL, int MODE, bool PF = false>
static int launch_q4k(int64_t n, int nb, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                      cudaStream_t s, PairMap pm = PairMap{}, int64_t pairs = 1) {
    const int splits = pm.ksplit > 1 ? pm.ksplit : 1;
    const int nw = pick_warps(splits > 1 ? (nb + splits - 1) / splits : nb);
    const size_t smem = sizeof(Q4KStage) * nw * NCOL + (splits > 1 ? 0 : sizeof(int4) * (size_t)NCOL * nb * 32 * (MODE == 1 ? 3 : 1));
    B200_REQUIRE(smem <= 200 * 1024, "mul_mat q4_K: k too large for the shared-memory exchange (%zu bytes)", smem);
    // the attribute belongs to the (function, device) pair: one flag per device
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemv: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<NCOL, MODE, PF>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done[dev] = true;
    }
    const int64_t tiles_n = pm.seg_count > 1 ? pm.seg_total : (n + TILE_ROWS - 1) / TILE_ROWS;
    B200_REQUIRE(pairs >= 1 && pairs <= 65535, "mul_mat_id: %lld (token, slot) pairs exceed one launch", (long long)pairs);
    return launch_pdl(gemv_q4_K_kernel<NCOL, MODE, PF>, dim3((unsigned)tiles_n, (unsigned)pairs, (unsigned)splits), dim3(nw * 32), smem, s,
                      tiles, acts, dst, lddst, n, nb, pm);
}

// B200_GEMV_PREFETCH=0 turns the prefetching form of the one-row Q4_K kernel off (for side-by-side measurements)
static bool gemv_prefetch_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMV_PREFETCH");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// B200_GEMV_ROW=0 keeps one-row Q4_K mat-muls on gemv_q4_K_kernel<1, 0> (for side-by-side measurements)
static bool gemv_row_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMV_ROW");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}
static int64_t gemv_stream_max_tiles();
template <bool PF>
static int launch_q4k_row_pf(dim3 grid, dim3 block, size_t smem, cudaStream_t s, const uint8_t *tiles, ActView acts, float *dst, int64_t n,
                             int nb, PairMap pm, const ActPrologue &pro) {
    switch (pro.mode) {
        case ACT_PRO_PLAIN: return launch_pdl(gemv_q4_K_row_kernel<PF, ACT_PRO_PLAIN>, grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
        case ACT_PRO_NORM: return launch_pdl(gemv_q4_K_row_kernel<PF, ACT_PRO_NORM>, grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
        case ACT_PRO_SILU: return launch_pdl(gemv_q4_K_row_kernel<PF, ACT_PRO_SILU>, grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
        default: return launch_pdl(gemv_q4_K_row_kernel<PF, ACT_PRO_NONE>, grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
    }
}
static int launch_q4k_row(int64_t n, int nb, const uint8_t *tiles, ActView acts, float *dst, cudaStream_t s, PairMap pm = PairMap{},
                          int64_t pairs = 1, const ActPrologue &pro = ActPrologue{}) {
    const int nw = pick_warps(nb);
    const size_t smem = sizeof(Q4KStage) * nw + (size_t)nb * 32 * sizeof(int4) + (size_t)nb * sizeof(float);
    B200_REQUIRE(smem <= 200 * 1024, "mul_mat q4_K: k too large for the shared-memory exchange (%zu bytes)", smem);
    const int64_t tiles_n = pm.seg_count > 1 ? pm.seg_total : (n + TILE_ROWS - 1) / TILE_ROWS;
    // long rows and at most a row tile per SM: the prefetching form (it needs the registers of a whole SM)
    const bool pf = nb > nw && tiles_n * pairs <= gemv_stream_max_tiles() && gemv_prefetch_enabled();
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemv: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<false, ACT_PRO_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<false, ACT_PRO_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<false, ACT_PRO_NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<false, ACT_PRO_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<true, ACT_PRO_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<true, ACT_PRO_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<true, ACT_PRO_NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_row_kernel<true, ACT_PRO_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done[dev] = true;
    }
    B200_REQUIRE(pairs >= 1 && pairs <= 65535, "mul_mat_id: %lld (token, slot) pairs exceed one launch", (long long)pairs);
    B200_REQUIRE(pro.mode == ACT_PRO_NONE || pairs == 1, "mul_mat_id takes no activation prologue");
    const dim3 grid((unsigned)tiles_n, (unsigned)pairs), block(nw * 32);
    if (pf) return launch_q4k_row_pf<true>(grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
    return launch_q4k_row_pf<false>(grid, block, smem, s, tiles, acts, dst, n, nb, pm, pro);
}

// B200_GEMV_KSPLIT=1 splits K over several CTAs per row tile for the few-tile decode mat-muls.  Measured it
// loses to the streaming kernel (4096 x 4096: 5.95 against 5.31 us; 4096 x 14336: 13.9 against 11.5 us), whose
// bulk copies already keep more bytes in flight per SM than four register-staged CTAs do; selectable only.
static bool gemv_ksplit_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMV_KSPLIT");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}
constexpr int KSPLIT_MAX_TILES = 1024;
// arrival counters of the K split, one per row tile, zero between launches: a file-scope device array (one
// zero-initialized copy per device that loads the module), addressed through cudaGetSymbolAddress
static __device__ int g_kcount_dev[KSPLIT_MAX_TILES];
static int *g_kcount[64] = {nullptr};
// One activation row, a matrix with fewer row tiles than the GPU has room for: split K over several CTAs per tile.
static int launch_q4k_ksplit(int splits, int64_t n, int nb, const uint8_t *tiles, ActView acts, float *dst, cudaStream_t s) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemv: device index %d out of range", dev);
    if (!g_kcount[dev]) {
        void *p = nullptr;
        B200_CUDA(cudaGetSymbolAddress(&p, g_kcount_dev));
        B200_REQUIRE(p != nullptr, "gemv: the device reported no address for the K-split counters");
        g_kcount[dev] = (int *)p;
    }
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    B200_REQUIRE(tiles_n <= KSPLIT_MAX_TILES, "gemv: %lld row tiles exceed the K-split counters", (long long)tiles_n);
    void *kx = nullptr;
    int rc = scratch_get_kx((size_t)tiles_n * nb * 32 * sizeof(int4), &kx);
    if (rc != B200_STATUS_SUCCESS) return rc;
    PairMap pm = PairMap{};
    pm.ksplit = splits;
    pm.kx = (int4 *)kx;
    pm.kcount = g_kcount[dev];
    return launch_q4k<1, 0>(n, nb, tiles, acts, dst, n, s, pm);
}

// One activation row against up to three Q4_K matrices of the same K (8x8 gemv chain): one launch whose CTAs
// walk the row tiles of all of them.  Every output element is computed exactly as by a launch of its own.
int launch_gemv_q4_K_multi(int count, const int64_t *n, const uint8_t *const *tiles, float *const *dst, int64_t k, ActView acts,
                           cudaStream_t s) {
    return launch_gemv_q4_K_row_fused(count, n, tiles, dst, k, acts, ActPrologue{}, s);
}

// The same with an activation prologue (see gemv_q4_K_row_kernel): acts.qs may be null when pro.mode != ACT_PRO_NONE;
// acts.addend / acts.sum (one matrix only) add the residual in the epilogue.
int launch_gemv_q4_K_row_fused(int count, const int64_t *n, const uint8_t *const *tiles, float *const *dst, int64_t k, ActView acts,
                               const ActPrologue &pro, cudaStream_t s) {
    B200_REQUIRE(count >= 1 && count <= 3, "mul_mat multi: %d matrices (1 to 3 fit one launch)", count);
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat multi: k = %lld must be a multiple of 256", (long long)k);
    B200_REQUIRE(count == 1 || acts.sum == nullptr, "mul_mat multi: the residual add goes with a single matrix");
    PairMap pm = PairMap{};
    pm.seg_count = count;
    pm.seg_end[1] = 0x7fffffff;   // "no third matrix"
    int64_t end = 0;
    for (int i = 0; i < count; i++) {
        B200_REQUIRE(n[i] > 0 && tiles[i] && dst[i], "mul_mat multi: matrix %d is empty or null", i);
        end += (n[i] + TILE_ROWS - 1) / TILE_ROWS;
        B200_REQUIRE(end < 0x7fffffffLL, "mul_mat multi: too many rows for one launch");
        if (i + 1 < count) pm.seg_end[i] = (int)end;
        if (i > 0) {
            pm.seg_tiles[i - 1] = tiles[i];
            pm.seg_dst[i - 1] = dst[i];
            pm.seg_n[i - 1] = n[i];
        }
    }
    pm.seg_total = (int)end;
    if (count == 1) pm.seg_count = 0;
    if (gemv_row_enabled() || pro.mode != ACT_PRO_NONE) return launch_q4k_row(n[0], (int)(k / GROUP_K), tiles[0], acts, dst[0], s, pm, 1, pro);
    return launch_q4k<1, 0>(n[0], (int)(k / GROUP_K), tiles[0], acts, dst[0], n[0], s, pm);
}

// ---------------------------------------------------------------------------
// Generic decode kernel for the other (type, route) pairs, see gemv_types.cuh.
// K is processed in windows of `win` groups so that the exchange array fits in
// shared memory; the chain threads keep their accumulators in registers across
// windows.  Chain threads: NCOL x CHAINS x 32, thread = (col, l, row).
// ---------------------------------------------------------------------------
template <class T, int NCOL, bool L2PF = false>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_generic_kernel(const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int win,
                    PairMap pm) {
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger();
    if (pm.ids) pdl_wait();
    if (!apply_pair(pm, tiles, acts, dst, lddst)) return;
    bool waited = pm.ids != nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    ActStage *stage = (ActStage *)smem + warp * NCOL;
    float *fin = (float *)(smem + sizeof(ActStage) * nwarps * NCOL);       // [NCOL][12][32]
    uint32_t *xch = (uint32_t *)(fin + NCOL * 12 * 32);                     // [NCOL][win][NW][32]
    const int64_t tile = blockIdx.x;
    const uint8_t *base = tiles + tile * (int64_t)nb * T::CHUNK;
    const int ct = threadIdx.x;  // chain thread id
    const bool is_chain = ct < NCOL * T::CHAINS * 32;
    const int c_col = ct / (T::CHAINS * 32), c_l = (ct >> 5) % T::CHAINS, c_row = ct & 31;
    float acc = 0.0f;

    for (int w0 = 0; w0 < nb; w0 += win) {
        const int wn = nb - w0 < win ? nb - w0 : win;
        for (int g = warp; g < wn; g += nwarps) {
            const int b = w0 + g;
            typename T::Regs regs;
            T::load(base + (int64_t)b * T::CHUNK, lane, regs);
            if (L2PF && g + nwarps < wn) {
                // the warp's next group of this window on its way from DRAM to L2 while this one is multiplied (no registers taken;
                // measured on the 8B step: 1.906 -> 1.882 ms per token; all the warp's later groups at once: 1.911)
                const uint8_t *nx = base + (int64_t)(b + nwarps) * T::CHUNK + lane * 16;
#pragma unroll
                for (int c = 0; c < T::CHUNK / 512; c++) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + c * 512));
            }
            if (!waited) { pdl_wait(); waited = true; }
#pragma unroll
            for (int col = 0; col < NCOL; col++) {
                const int8_t *aq = acts.qs + (int64_t)col * acts.k + (int64_t)b * 256;
                if (lane < 16) {
                    stage[col].q[lane] = *(const uint4 *)(aq + lane * 16);
                } else if (T::ACT_Q8K) {
                    if (lane < 24) {
                        const int j = lane - 16;
                        const short2 s2 = *(const short2 *)(acts.bsums + (int64_t)col * (acts.k / 16) + (int64_t)b * 16 + 2 * j);
                        stage[col].aux[2 * j] = s2.x;
                        stage[col].aux[2 * j + 1] = s2.y;
                    }
                } else if (lane < 24) {
                    const int blk = lane - 16;  // sum of the block's 32 quants
                    const uint4 y0 = *(const uint4 *)(aq + blk * 32), y1 = *(const uint4 *)(aq + blk * 32 + 16);
                    int sum = 0;
                    sum = dp4(0x01010101u, y0.x, sum); sum = dp4(0x01010101u, y0.y, sum);
                    sum = dp4(0x01010101u, y0.z, sum); sum = dp4(0x01010101u, y0.w, sum);
                    sum = dp4(0x01010101u, y1.x, sum); sum = dp4(0x01010101u, y1.y, sum);
                    sum = dp4(0x01010101u, y1.z, sum); sum = dp4(0x01010101u, y1.w, sum);
                    stage[col].aux[8 + blk] = sum;
                }
            }
            __syncwarp();
#pragma unroll
            for (int col = 0; col < NCOL; col++)
                T::compute(regs, stage[col], xch + ((int64_t)(col * win + g) * T::NW) * 32 + lane);
            __syncwarp();
        }
        if (!waited) { pdl_wait(); waited = true; }
        __syncthreads();
        if (is_chain) {
            for (int g = 0; g < wn; g++)
                T::chain(acc, xch + ((int64_t)(c_col * win + g) * T::NW) * 32 + c_row, c_l, acts, c_col, w0 + g);
        }
        __syncthreads();
    }
    const int64_t row0 = tile * TILE_ROWS;
    if (T::CHAINS == 1) {
        if (is_chain && row0 + c_row < n) {
            dst[(int64_t)c_col * lddst + row0 + c_row] = acc;
            if (acts.sum && c_col == 0) acts.sum[row0 + c_row] = __fadd_rn(acc, acts.addend[row0 + c_row]);
        }
    } else {
        // hsum8 of the eight lane accumulators: crates/ggml/src/vec_dot.rs:564-572
        if (is_chain) fin[(c_col * 12 + c_l) * 32 + c_row] = acc;
        __syncthreads();
        if (ct < NCOL * 32) {
            const int col = ct >> 5, r = ct & 31;
            const float *a = fin + col * 12 * 32 + r;
            const float r0 = __fadd_rn(a[4 * 32], a[0]), r1 = __fadd_rn(a[5 * 32], a[32]);
            const float r2 = __fadd_rn(a[6 * 32], a[2 * 32]), r3 = __fadd_rn(a[7 * 32], a[3 * 32]);
            float v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
            if (T::CHAINS == 12) {
                // the four min lanes of the Q4_K row dot: (m0 + m2) + (m1 + m3), added last
                const float m01 = __fadd_rn(__fadd_rn(a[8 * 32], a[10 * 32]), __fadd_rn(a[9 * 32], a[11 * 32]));
                v = __fadd_rn(v, m01);
            }
            if (row0 + r < n) {
                dst[(int64_t)col * lddst + row0 + r] = v;
                if (acts.sum && col == 0) acts.sum[row0 + r] = __fadd_rn(v, acts.addend[row0 + r]);
            }
        }
    }
}

constexpr size_t GEMV_SMEM_LIMIT = 200 * 1024;

template <class T, int NCOL>
static int launch_generic(int64_t n, int nb, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                          cudaStream_t s, PairMap pm = PairMap{}, int64_t pairs = 1) {
    const size_t per_group = (size_t)NCOL * T::NW * 32 * 4;
    // warps: enough chain threads, and an even split of the groups when possible
    int nw = pick_warps(nb);
    const int min_warps = NCOL * T::CHAINS;
    if (nw < min_warps) nw = min_warps;
    const size_t fixed = sizeof(ActStage) * nw * NCOL + (size_t)NCOL * 12 * 32 * 4;
    int win = (int)((GEMV_SMEM_LIMIT - fixed) / per_group);
    if (win > nb) win = nb;
    if (win > nw && win % nw) win -= win % nw;  // whole rounds of warps per window
    B200_REQUIRE(win >= 1, "gemv: shared memory too small for one group");
    const size_t smem = fixed + per_group * win;
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemv: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemv_generic_kernel<T, NCOL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)GEMV_SMEM_LIMIT));
        attr_done[dev] = true;
    }
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    B200_REQUIRE(pairs >= 1 && pairs <= 65535, "mul_mat_id: %lld (token, slot) pairs exceed one launch", (long long)pairs);
    // Q6_K row dot over long rows (the ffn_down of the Q6_K layers: four groups per warp): with the L2 prefetch of the next group;
    // B200_GEMV_PREFETCH=0 turns it off
    if (std::is_same<T, TraitsQ6K>::value && NCOL == 1 && nb > nw && gemv_prefetch_enabled()) {
        static bool pf_attr_done[64] = {false};
        if (!pf_attr_done[dev]) {
            B200_CUDA(cudaFuncSetAttribute(gemv_generic_kernel<T, NCOL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMV_SMEM_LIMIT));
            pf_attr_done[dev] = true;
        }
        return launch_pdl(gemv_generic_kernel<T, NCOL, true>, dim3((unsigned)tiles_n, (unsigned)pairs), dim3(nw * 32), smem, s, tiles, acts, dst, lddst, n,
                          nb, win, pm);
    }
    return launch_pdl(gemv_generic_kernel<T, NCOL>, dim3((unsigned)tiles_n, (unsigned)pairs), dim3(nw * 32), smem, s,
                      tiles, acts, dst, lddst, n, nb, win, pm);
}

// columns in passes of at most MAXC; the weights are re-read per pass (decode shapes only)
template <class T, int MAXC>
static int run_generic(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                       cudaStream_t s) {
    const int nb = (int)(k / GROUP_K);
    for (int64_t c0 = 0; c0 < m; c0 += MAXC) {
        const int nc = (int)(m - c0 < MAXC ? m - c0 : MAXC);
        ActView a = acts;
        a.qs += c0 * k;
        if (a.d) a.d += c0 * nb;
        if (a.bsums) a.bsums += c0 * (k / 16);
        if (a.dh) a.dh += c0 * (k / 32);
        float *o = dst + c0 * lddst;
        int rc;
        if (MAXC >= 2 && nc == 2) rc = launch_generic<T, (MAXC >= 2 ? 2 : 1)>(n, nb, tiles, a, o, lddst, s);
        else if (nc == 1) rc = launch_generic<T, 1>(n, nb, tiles, a, o, lddst, s);
        else rc = launch_generic<T, (MAXC >= 2 ? 2 : 1)>(n, nb, tiles, a, o, lddst, s);
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    return B200_STATUS_SUCCESS;
}

// Which kernel a one-row Q4_K mat-mul of at most one row tile per SM takes.  Timed inside a replayed CUDA graph (the
// way a decode step runs them) the register-staged kernel wins on every shape: 4096 x 4096 3.3 against 4.3 us,
// 4096 x 14336 10.2 against 11.4 us; the bulk-copy streaming kernel only looked faster when a host loop issued the
// launches and the host's launch rate was what was being measured.  B200_GEMV_STREAM=1 selects the streaming kernel
// (read once), and so does the wait test hook while it is armed.
bool gemv_stream_forced();   // gemv_stream.cu
static bool gemv_stream_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMV_STREAM");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1 || gemv_stream_forced();
}

// B200_GEMM_MMA=0 keeps prompt batches on the column-pass kernels (for side-by-side measurements)
constexpr int64_t GEMM_MMA_MIN_COLS = 8;
static bool gemm_mma_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMM_MMA");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// B200_GEMM_TCGEN05=0 keeps Q4_K prompt batches on the mma.sync kernel; batches narrower than one
// 32-column MMA tile stay there too
constexpr int64_t GEMM_TCGEN05_MIN_COLS = 32;
static bool gemm_tcgen05_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMM_TCGEN05");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// B200_STREAM_TILES_MULT=<m>: matrices of up to m row tiles per SM take the streaming kernel (default 1)
static int gemv_stream_tiles_mult() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_STREAM_TILES_MULT");
        v = e ? atoi(e) : 1;
        if (v < 1) v = 1;
    }
    return v;
}
static int64_t gemv_stream_max_tiles() {
    static int sms[64] = {0};   // per device: a process may drive GPUs with different SM counts
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (sms[dev] == 0 && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 0;
    return (int64_t)sms[dev] * gemv_stream_tiles_mult();
}

// whether launch_gemv takes (type, route, m activation rows) to a few-rows kernel, which can add a tensor to its result as it stores it
bool gemv_rows_add_fusable(int type, int route, int64_t m) {
    if (!(m >= GEMM_MMA_MIN_COLS && m < 32 && gemm_mma_enabled() && gemm_small_multi_enabled())) return false;
    return (type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK && m % 4 == 0) || (type == B200_TYPE_Q6_K && route == B200_ROUTE_TILED);
}

// Several Q4_K matrices of one row length against the same activation rows: one launch of the fast-numerics prompt kernel
// where each of them would take it by itself (the same kernel and tolerance; its CTAs cut the tiles' f32 sums in other
// places than separate launches would), separate launches otherwise.
int launch_gemv_rows_multi(int type, int route, int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                           const int64_t *lddst, cudaStream_t s) {
    const char *fe = getenv("B200_GEMM_FAST");
    const bool whole = route == B200_ROUTE_TILED || (route == B200_ROUTE_REPACK && m % 4 == 0);   // no tail rows on another chain
    int64_t rows = 0;
    for (int e = 0; e < count; e++) rows += n[e];
    if (count > 1 && type == B200_TYPE_Q4_K && whole && (rows >= 2048 || (fe && fe[0] == '2')) && m >= GEMM_FAST_MIN_COLS && m >= GEMM_TCGEN05_MIN_COLS && gemm_mma_enabled() && gemm_tcgen05_enabled() &&
        gemm_tcgen05_f16_choice() < 0 && numerics_mode() == 1 && !no_scratch_mode() && !(fe && fe[0] == '0'))
        return launch_gemm_kq_fast_multi(type, count, n, k, m, tiles, acts, dst, lddst, s);
    // a batched decode step's rows (8 to 31, a multiple of 4): the few-rows kernel takes the matrices as one grid, the same
    // CTAs and chains as separate launches (bit-identical)
    if (count > 1 && count <= 3 && type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK && m % 4 == 0 && m >= GEMM_MMA_MIN_COLS && m < 32 && gemm_mma_enabled() &&
        gemm_small_multi_enabled())
        return launch_gemm_small_multi(count, n, k, m, tiles, acts, dst, lddst, s);
    for (int e = 0; e < count; e++) {
        int rc = launch_gemv(type, route, n[e], k, m, tiles[e], acts, dst[e], lddst[e], s);
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    return B200_STATUS_SUCCESS;
}

int launch_gemv(int type, int route, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst,
                int64_t lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemv: k = %lld must be a multiple of 256", (long long)k);
    const int nb = (int)(k / GROUP_K);
    // the bulk-copy streaming kernel wins while every CTA has at most one row tile (no second wave to
    // overlap); beyond that the register-staged kernel with two CTAs per SM keeps more warps busy
    if (type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK && m == 1 && gemv_ksplit_enabled() && !no_scratch_mode() && nb >= 8 &&
        (n + TILE_ROWS - 1) / TILE_ROWS <= gemv_stream_max_tiles()) {
        // at most one row tile per SM: four CTAs per tile (two for short rows), each a quarter of K
        const int splits = nb >= 16 ? 4 : 2;
        return launch_q4k_ksplit(splits, n, nb, tiles, acts, dst, s);
    }
    if (type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK && m == 1 && gemv_stream_enabled() &&
        (n + TILE_ROWS - 1) / TILE_ROWS <= gemv_stream_max_tiles())
        return launch_gemv_q4_K_stream(n, k, tiles, acts, dst, s);
    if (type == B200_TYPE_Q4_K && (route == B200_ROUTE_REPACK || route == B200_ROUTE_TILED)) {
        // REPACK: the caller quantized the first m - m % 4 rows with the 4x8 rule (gemm chain) and the
        // tail rows the plain way (gemv chain), exactly as crates/ggml/src/compute.rs:5322-5447 does.
        const int64_t m4 = route == B200_ROUTE_REPACK ? m - m % 4 : m;
        const int maxc_main = route == B200_ROUTE_REPACK ? 2 : 3;
        int64_t c_start = 0;
        if (m4 >= GEMM_MMA_MIN_COLS && gemm_mma_enabled()) {
            // enough activation rows to fill tensor-core patches: same chains, integer dots by mma
            const int mode = route == B200_ROUTE_REPACK ? 1 : 2;
            int rc = m4 >= GEMM_TCGEN05_MIN_COLS && gemm_tcgen05_enabled() ? launch_gemm_tcgen05(mode, n, k, m4, tiles, acts, dst, lddst, s)
                                                                           : launch_gemm_mma(mode, n, k, m4, tiles, acts, dst, lddst, s);
            if (rc != B200_STATUS_SUCCESS) return rc;
            c_start = m4;
        }
        for (int64_t c0 = c_start; c0 < m;) {
            const bool main_part = c0 < m4;
            const int64_t end = main_part ? m4 : m;
            const int maxc = main_part ? maxc_main : 3;
            const int nc = (int)(end - c0 < maxc ? end - c0 : maxc);
            ActView a = acts;
            a.qs += c0 * k;
            a.d += c0 * nb;
            a.bsums += c0 * (k / 16);
            float *o = dst + c0 * lddst;
            int rc;
            if (route == B200_ROUTE_TILED) {
                rc = nc == 1 ? launch_q4k<1, 2>(n, nb, tiles, a, o, lddst, s)
                   : nc == 2 ? launch_q4k<2, 2>(n, nb, tiles, a, o, lddst, s)
                             : launch_q4k<3, 2>(n, nb, tiles, a, o, lddst, s);
            } else if (main_part) {
                rc = nc == 1 ? launch_q4k<1, 1>(n, nb, tiles, a, o, lddst, s) : launch_q4k<2, 1>(n, nb, tiles, a, o, lddst, s);
            } else {
                // one activation row, long rows and at most a row tile per SM: the prefetching form
                const bool pf = nc == 1 && nb > GEMV_MAX_WARPS && (n + TILE_ROWS - 1) / TILE_ROWS <= gemv_stream_max_tiles() && gemv_prefetch_enabled();
                rc = nc == 1 && m == 1 && gemv_row_enabled() ? launch_q4k_row(n, nb, tiles, a, o, s)
                   : nc == 1 ? (pf ? launch_q4k<1, 0, true>(n, nb, tiles, a, o, lddst, s) : launch_q4k<1, 0>(n, nb, tiles, a, o, lddst, s))
                   : nc == 2 ? launch_q4k<2, 0>(n, nb, tiles, a, o, lddst, s)
                             : launch_q4k<3, 0>(n, nb, tiles, a, o, lddst, s);
            }
            if (rc != B200_STATUS_SUCCESS) return rc;
            c0 += nc;
        }
        return B200_STATUS_SUCCESS;
    }
    // 32 activation rows and up: tcgen05 int8 kernels.  Q6_K (tiled chain, on request), Q4_0 and MXFP4 (8x8 gemm chain) keep the CPU
    // routes' bits; Q8_0's tensor-core form adds whole 32-element dots where the CPU adds eight 4-element lanes, so it
    // serves the fast numerics mode only.  The 32-element-block types take it from 8 rows on (their only alternative
    // re-reads the weights once per two activation rows).
    if (gemm_tcgen05_enabled() && gemm_mma_enabled()) {
        // fast numerics: Q6_K prompt batches on the f16 tensor-core kernel with one accumulator per super-block (within 1e-5
        // of sum |w x|), from 2048 weight rows (measured with 512 activation rows: 4096 x 14336 424 -> 218 us, 14336 x 4096
        // 382 -> 204 us, but 1024 x 4096 48 -> 90 us: eight row blocks leave its producer warps nothing to hide behind);
        // B200_GEMM_FAST=0 keeps the exact kernels, =2 lifts the row limit (read per call)
        const char *fe = getenv("B200_GEMM_FAST");
        if (type == B200_TYPE_Q6_K && route == B200_ROUTE_TILED && m >= GEMM_FAST_MIN_COLS && numerics_mode() == 1 && !no_scratch_mode() &&
            (n >= 2048 || (fe && fe[0] == '2'))) {
            if (!(fe && fe[0] == '0')) return launch_gemm_kq_fast(type, n, k, m, tiles, acts, dst, lddst, s);
        }
        // Q6_K: the two-plane tcgen05 kernel gives the same bits as the mma.sync kernel below but measured slower
        // (107-114 against 156-170 TOP/s on 14336 x 4096 with 512 / 2048 rows: its operand split is the bottleneck),
        // so it runs only when asked for: B200_Q6K_TCGEN05=1, read per call
        if (type == B200_TYPE_Q6_K && route == B200_ROUTE_TILED && m >= GEMM_TCGEN05_MIN_COLS) {
            const char *e = getenv("B200_Q6K_TCGEN05");
            if (e && e[0] == '1') return launch_gemm_tcgen05_i8(type, n, k, m, tiles, acts, dst, lddst, s);
        }
        if ((type == B200_TYPE_Q4_0 || type == B200_TYPE_MXFP4) && route == B200_ROUTE_REPACK && m >= GEMM_MMA_MIN_COLS)
            return launch_gemm_tcgen05_i8(type, n, k, m, tiles, acts, dst, lddst, s);
        if (type == B200_TYPE_Q8_0 && route == B200_ROUTE_ROWDOT && m >= GEMM_MMA_MIN_COLS && numerics_mode() == 1)
            return launch_gemm_tcgen05_i8(type, n, k, m, tiles, acts, dst, lddst, s);
    }
    if (type == B200_TYPE_Q6_K && route == B200_ROUTE_TILED && m >= GEMM_MMA_MIN_COLS && gemm_mma_enabled())
        return launch_gemm_mma(6, n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_Q6_K && route == B200_ROUTE_TILED) return run_generic<TraitsQ6KTiled, 2>(n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_Q4_K && route == B200_ROUTE_ROWDOT) return run_generic<TraitsQ4KRowDot, 1>(n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_Q6_K && route == B200_ROUTE_ROWDOT) return run_generic<TraitsQ6K, 1>(n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_Q8_0 && route == B200_ROUTE_ROWDOT) return run_generic<TraitsQ8_0, 1>(n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_Q4_0 && route == B200_ROUTE_REPACK) return run_generic<TraitsB32<false>, 2>(n, k, m, tiles, acts, dst, lddst, s);
    if (type == B200_TYPE_MXFP4 && route == B200_ROUTE_REPACK) return run_generic<TraitsB32<true>, 2>(n, k, m, tiles, acts, dst, lddst, s);
    B200_REQUIRE(false, "mul_mat: no kernel yet for weight type %d with route %d (m = %lld)", type, route, (long long)m);
}

// B200_MMID_GROUPED=0 keeps MUL_MAT_ID on one CTA set per (token, slot) pair (for side-by-side measurements)
static bool mmid_grouped_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_MMID_GROUPED");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// rows routed to each expert (for the tiled / row-dot split of K-quant experts)
__global__ void count_expert_rows_kernel(const int32_t *ids, int64_t n_pairs, int n_expert, int *counts) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = ids[i];
    if (e >= 0 && e < n_expert) atomicAdd(&counts[e], 1);
}

// MUL_MAT_ID: crates/ggml/src/compute.rs:1917-2202.  Experts whose row count is a multiple of 8
// run the 8x8 gemv chain per pair (MXFP4, Q4_0, Q4_K); other K-quant experts take the tiled chain
// when at least 8 rows were routed to them and the row dot otherwise; the rest is the row dot.
int launch_mul_mat_id(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok, int64_t n_ids,
                      const uint8_t *tiles, ActView acts, const int32_t *ids, float *dst, int *counts, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat_id: k = %lld must be a multiple of 256", (long long)k);
    const int nb = (int)(k / GROUP_K);
    const int64_t pairs = n_tok * n_ids;
    if (pairs == 0 || n == 0) return B200_STATUS_SUCCESS;
    PairMap pm{};
    pm.ids = ids;
    pm.n_ids = (int)n_ids;
    pm.ne11 = (int)ne11;
    pm.n_expert = (int)n_expert;
    pm.expert_bytes = (int64_t)((n + TILE_ROWS - 1) / TILE_ROWS) * nb * chunk_bytes(type);
    pm.counts = nullptr;
    pm.min_count = 0;
    pm.max_count = 0x7fffffff;
    const bool repack = n % 8 == 0;
    // enough pairs to fill tensor-core tiles: grouped by expert, every expert's weights read once (same per-block chain,
    // same bits as the per-pair kernels below)
    if ((type == B200_TYPE_MXFP4 || type == B200_TYPE_Q4_0) && repack && pairs >= 64 && mmid_grouped_enabled() && gemm_tcgen05_enabled())
        return launch_mul_mat_id_grouped(type, n, k, n_expert, ne11, n_tok, n_ids, tiles, acts, ids, dst, counts, s);
    if (type == B200_TYPE_MXFP4 && repack) return launch_generic<TraitsB32<true>, 1>(n, nb, tiles, acts, dst, n, s, pm, pairs);
    if (type == B200_TYPE_Q4_0 && repack) return launch_generic<TraitsB32<false>, 1>(n, nb, tiles, acts, dst, n, s, pm, pairs);
    if (type == B200_TYPE_Q4_K && repack)
        return gemv_row_enabled() ? launch_q4k_row(n, nb, tiles, acts, dst, s, pm, pairs) : launch_q4k<1, 0>(n, nb, tiles, acts, dst, n, s, pm, pairs);
    if (type == B200_TYPE_Q8_0) return launch_generic<TraitsQ8_0, 1>(n, nb, tiles, acts, dst, n, s, pm, pairs);
    if (type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K) {
        B200_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * n_expert, s));
        count_expert_rows_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, s>>>(ids, pairs, (int)n_expert, counts);
        B200_CUDA(cudaGetLastError());
        pm.counts = counts;
        PairMap lo = pm, hi = pm;
        lo.max_count = 7;
        hi.min_count = 8;
        int rc;
        if (type == B200_TYPE_Q4_K) {
            rc = launch_q4k<1, 2>(n, nb, tiles, acts, dst, n, s, hi, pairs);
            if (rc == B200_STATUS_SUCCESS) rc = launch_generic<TraitsQ4KRowDot, 1>(n, nb, tiles, acts, dst, n, s, lo, pairs);
        } else {
            rc = launch_generic<TraitsQ6KTiled, 1>(n, nb, tiles, acts, dst, n, s, hi, pairs);
            if (rc == B200_STATUS_SUCCESS) rc = launch_generic<TraitsQ6K, 1>(n, nb, tiles, acts, dst, n, s, lo, pairs);
        }
        return rc;
    }
    B200_REQUIRE(false, "mul_mat_id: no kernel for expert type %d with %lld rows per expert", type, (long long)n);
}

}  // namespace b200
