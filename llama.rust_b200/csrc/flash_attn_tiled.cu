// FLASH_ATTN_EXT, prefill-shaped (64 query rows or more): the arithmetic of the
// CPU path's tiled kernel (crates/ggml/src/flash_attn.rs:1111-1361), exactly.
//
// One CTA per (head, 64-row query tile) walks the KV range in tiles of 64:
//   KQ   = Q_tile * K_tile^T      one f32 FMA chain per element, d ascending
//   KQ  *= scale; softcap; -inf padding; += mask (valid rows)
//   per row: tile maximum, rescale of the running row by libm expf when the
//            maximum grows, P = v_expf(KQ - M) (the AVX512 polynomial, f32 FMAs,
//            single-rounded scalef), S += f64 sum of the 16-lane reduce trees
//   VKQ += P * V_tile              one f32 FMA chain per element, kv ascending
// followed by sinks, S_inv and the store.  Everything is CUDA-core f32 so the
// result is bit-comparable with the CPU; the tensor-core version is a separate
// fast mode.
#include "common.cuh"
#include "fa_math.cuh"

namespace b200 {

constexpr int QT = 64, KT = 64;

struct TiledDims {
    int dk, dv, T, H, H_kv;
    int64_t n_kv;
};

// Shared memory (floats): qT[dk][64] | kT[dk][64] | v[64][dv] | p[64 kv][64 q] | mask[64 q][64 kv]
// 256 threads.  Register blocks: KQ 4 q x 4 kv per thread, VKQ 4 q x (dv/16) d per thread.
template <int DK, int DV>
__global__ void __launch_bounds__(256)
fa_tiled_kernel(b200_flash_attn_args a, TiledDims d, float kq_scale) {
    extern __shared__ __align__(16) float tsm[];
    float *qT = tsm;                    // [DK][QT]
    float *kT = qT + DK * QT;           // [DK][KT]
    float *vS = kT + DK * KT;           // [KT][DV]
    float *pS = vS + KT * DV;           // [KT][QT]   (KQ, then P; kv-major so the PV loop reads float4 over q)
    float *mS = pS + KT * QT;           // [QT][KT]
    __shared__ float rowM[QT], rowS[QT], rowScale[QT];
    __shared__ int rowSkip[QT];
    __shared__ int can_skip_flag;
    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int64_t t0 = (int64_t)blockIdx.x * QT;
    const int tile_rows = d.T - t0 < QT ? (int)(d.T - t0) : QT;
    const int hkv = h / (d.H / d.H_kv);
    const uint8_t *kb = (const uint8_t *)a.k + (int64_t)hkv * a.k_nb2;
    const uint8_t *vb = (const uint8_t *)a.v + (int64_t)hkv * a.v_nb2;

    float slope = 1.0f;
    if (a.max_bias > 0.0f) {   // crates/ggml/src/flash_attn.rs:356-370
        const unsigned nl2 = 1u << (31 - __clz((unsigned)d.H));
        const float m0 = powf(2.0f, -a.max_bias / (float)nl2), m1 = powf(2.0f, -(a.max_bias / 2.0f) / (float)nl2);
        const float base = (unsigned)h < nl2 ? m0 : m1;
        const int ex = (unsigned)h < nl2 ? h + 1 : 2 * (h - (int)nl2) + 1;
        float acc = 1.0f, bb = base;
        for (int e2 = ex; e2 > 0; e2 >>= 1) {
            if (e2 & 1) acc = __fmul_rn(acc, bb);
            bb = __fmul_rn(bb, bb);
        }
        slope = acc;
    }

    // Q tile, transposed, zero-padded rows
    for (int i = tid; i < QT * DK; i += 256) {
        const int tq = i / DK, e = i % DK;
        float v = 0.0f;
        if (tq < tile_rows)
            v = ((const float *)((const uint8_t *)a.q + (t0 + tq) * a.q_nb1 + (int64_t)h * a.q_nb2))[e];
        qT[e * QT + tq] = v;
    }
    for (int i = tid; i < KT * DV; i += 256) vS[i] = 0.0f;
    if (tid < QT) { rowM[tid] = -INFINITY; rowS[tid] = 0.0f; }
    // VKQ accumulators: thread owns q rows 4*(tid/16) .. +3 and d = (tid%16) + 16*j
    constexpr int DJ = DV / 16;
    float acc[4][DJ];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < DJ; j++) acc[i][j] = 0.0f;
    const int q4 = (tid / 16) * 4, dlane = tid % 16;
    // KQ block: q rows 4*(tid/16).., kv columns 4*(tid%16)..
    const int kv4 = (tid % 16) * 4;
    __syncthreads();

    for (int64_t ic = 0; ic < d.n_kv; ic += KT) {
        const int kv_tile = d.n_kv - ic < KT ? (int)(d.n_kv - ic) : KT;
        // mask tile and the all-masked skip (flash_attn.rs:1181-1203)
        if (a.mask) {
            if (tid == 0) can_skip_flag = 1;
            __syncthreads();
            bool any = false;
            for (int i = tid; i < tile_rows * KT; i += 256) {
                const int tq = i / KT, tk = i % KT;
                float mv = -INFINITY;
                if (tk < kv_tile) {
                    const __half mh = ((const __half *)((const uint8_t *)a.mask + (t0 + tq) * a.mask_nb1))[ic + tk];
                    mv = __fmul_rn(slope, __half2float(mh));
                    if (mv != -INFINITY) any = true;
                }
                mS[tq * KT + tk] = mv;
            }
            if (any) can_skip_flag = 0;
            __syncthreads();
            const int skip_tile = can_skip_flag;
            __syncthreads();   // everyone has read the flag before thread 0 may reset it
            if (skip_tile) continue;
        }
        // K tile, transposed to [d][kv]; columns past kv_tile keep stale data (overwritten by -inf below)
        for (int i = tid; i < kv_tile * (DK / 8); i += 256) {
            const int tk = i / (DK / 8), c = i % (DK / 8);
            const uint4 raw = *(const uint4 *)(kb + (ic + tk) * a.k_nb1 + c * 16);
            const __half2 *hp = (const __half2 *)&raw;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(hp[j]);
                kT[(c * 8 + 2 * j) * KT + tk] = f.x;
                kT[(c * 8 + 2 * j + 1) * KT + tk] = f.y;
            }
        }
        // V tile to f32 [kv][d]; rows past kv_tile keep the previous tile's values (multiplied by P = 0)
        for (int i = tid; i < kv_tile * (DV / 8); i += 256) {
            const int tk = i / (DV / 8), c = i % (DV / 8);
            const uint4 raw = *(const uint4 *)(vb + (ic + tk) * a.v_nb1 + c * 16);
            const __half2 *hp = (const __half2 *)&raw;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float2 f = __half22float2(hp[j]);
                vS[tk * DV + c * 8 + 2 * j] = f.x;
                vS[tk * DV + c * 8 + 2 * j + 1] = f.y;
            }
        }
        __syncthreads();
        // KQ = Q K^T: chains over d ascending
        {
            float c[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) c[i][j] = 0.0f;
#pragma unroll 4
            for (int e = 0; e < DK; e++) {
                const float4 qv = *(const float4 *)(qT + e * QT + q4);
                const float4 kv = *(const float4 *)(kT + e * KT + kv4);
                const float qa[4] = {qv.x, qv.y, qv.z, qv.w}, ka[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) c[i][j] = __fmaf_rn(qa[i], ka[j], c[i][j]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int tq = q4 + i, tk = kv4 + j;
                    float s = __fmul_rn(c[i][j], kq_scale);
                    if (a.logit_softcap != 0.0f) s = __fmul_rn(a.logit_softcap, tanhf(s));
                    if (tk >= kv_tile) s = -INFINITY;
                    if (a.mask && tq < tile_rows) s = __fadd_rn(s, mS[tq * KT + tk]);
                    pS[tk * QT + tq] = s;
                }
        }
        __syncthreads();
        // per-row maximum and rescale factor (threads 0..63 = rows)
        if (tid < QT) {
            float mx = -INFINITY;
            for (int tk = 0; tk < KT; tk++) {
                const float v = pS[tk * QT + tid];
                mx = mx > v ? mx : v;
            }
            if (mx == -INFINITY) {
                rowSkip[tid] = 1;
                rowScale[tid] = 1.0f;
            } else {
                rowSkip[tid] = 0;
                const float m_old = rowM[tid];
                const float m_new = m_old > mx ? m_old : mx;
                float ms = 1.0f;
                if (m_new > m_old) {
                    ms = libm_expf(__fsub_rn(m_old, m_new));
                    rowS[tid] = __fmul_rn(rowS[tid], ms);
                }
                rowScale[tid] = ms;
                rowM[tid] = m_new;
            }
        }
        __syncthreads();
        // P = v_expf(KQ - M) for live rows, 0 for skipped rows
        for (int i = tid; i < QT * KT; i += 256) {
            const int tk = i / QT, tq = i % QT;
            pS[i] = rowSkip[tq] ? 0.0f : v_expf(__fsub_rn(pS[tk * QT + tq], rowM[tq]));
        }
        __syncthreads();
        // row sums: four 16-lane reduce trees per row, added in f64 (flash_attn.rs:997-1049)
        if (tid < QT && !rowSkip[tid]) {
            double sum = 0.0;
            for (int g = 0; g < 4; g++) {
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = pS[(16 * g + j) * QT + tid];
                float t3[8];
#pragma unroll
                for (int j = 0; j < 8; j++) t3[j] = __fadd_rn(v[8 + j], v[j]);
                const float t60 = __fadd_rn(t3[4], t3[0]), t61 = __fadd_rn(t3[5], t3[1]);
                const float t62 = __fadd_rn(t3[6], t3[2]), t63 = __fadd_rn(t3[7], t3[3]);
                sum = __dadd_rn(sum, (double)__fadd_rn(__fadd_rn(t60, t62), __fadd_rn(t61, t63)));
            }
            rowS[tid] = __double2float_rn(__dadd_rn((double)rowS[tid], sum));
        }
        // VKQ: rescale, then += P V with chains over kv ascending
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float ms = rowScale[q4 + i];
            if (ms != 1.0f)
#pragma unroll
                for (int j = 0; j < DJ; j++) acc[i][j] = __fmul_rn(acc[i][j], ms);
        }
#pragma unroll 4
        for (int tk = 0; tk < KT; tk++) {
            const float4 pv = *(const float4 *)(pS + tk * QT + q4);
            const float pa[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int j = 0; j < DJ; j++) {
                const float vv = vS[tk * DV + dlane + 16 * j];
#pragma unroll
                for (int i = 0; i < 4; i++) acc[i][j] = __fmaf_rn(pa[i], vv, acc[i][j]);
            }
        }
        __syncthreads();
    }
    // sinks (valid rows), S_inv, store (flash_attn.rs:1320-1356)
    __syncthreads();
    if (a.sinks && tid < QT) {
        const float sv = a.sinks[h];
        float ms = 1.0f, vs = 1.0f;
        if (sv > rowM[tid]) ms = libm_expf(__fsub_rn(rowM[tid], sv));
        else vs = libm_expf(__fsub_rn(sv, rowM[tid]));
        rowScale[tid] = ms;
        rowS[tid] = __fmaf_rn(rowS[tid], ms, vs);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int tq = q4 + i;
        if (tq >= tile_rows) continue;
        const float S = rowS[tq];
        const float s_inv = S == 0.0f ? 0.0f : __fdiv_rn(1.0f, S);
        float *o = a.dst + ((t0 + tq) * d.H + h) * DV;
#pragma unroll
        for (int j = 0; j < DJ; j++) {
            float v = acc[i][j];
            if (a.sinks && rowScale[tq] != 1.0f) v = __fmul_rn(v, rowScale[tq]);
            o[dlane + 16 * j] = __fmul_rn(v, s_inv);
        }
    }
}

template <int DK, int DV>
static int launch_tiled(const b200_flash_attn_args *a, const TiledDims &d, float kq_scale, cudaStream_t s) {
    const size_t smem = (size_t)(DK * QT + DK * KT + KT * DV + KT * QT + QT * KT) * 4;
    static bool done[64] = {false};   // the attribute belongs to the (function, device) pair
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "flash_attn_ext: device index %d out of range", dev);
    if (!done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(fa_tiled_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        done[dev] = true;
    }
    dim3 grid((unsigned)((d.T + QT - 1) / QT), (unsigned)d.H);
    fa_tiled_kernel<DK, DV><<<grid, 256, smem, s>>>(*a, d, kq_scale);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

int flash_attn_faithful_tiled(const b200_flash_attn_args *a, cudaStream_t s) {
    TiledDims d;
    d.dk = (int)a->dk; d.dv = (int)a->dv; d.T = (int)a->n_tok; d.H = (int)a->n_head; d.H_kv = (int)a->n_head_kv;
    d.n_kv = a->n_kv;
    B200_REQUIRE(d.H <= 65535, "flash_attn_ext: too many heads for one launch");
    const float kq_scale = a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
    if (d.dk == 128 && d.dv == 128) return launch_tiled<128, 128>(a, d, kq_scale, s);
    if (d.dk == 64 && d.dv == 64) return launch_tiled<64, 64>(a, d, kq_scale, s);
    if (d.dk == 64 && d.dv == 128) return launch_tiled<64, 128>(a, d, kq_scale, s);
    if (d.dk == 128 && d.dv == 64) return launch_tiled<128, 64>(a, d, kq_scale, s);
    B200_REQUIRE(false, "flash_attn_ext: head sizes (%d, %d) are not supported by the tiled path", d.dk, d.dv);
}

}  // namespace b200
