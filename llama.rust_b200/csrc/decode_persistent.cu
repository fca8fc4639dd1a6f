// One-token decode step as ONE persistent kernel.
//
// At one token a decoder layer is a dozen kernels of a few microseconds each: every one of them pays a launch, a ramp
// of its memory pipeline and a drain, and the weights (the only real traffic) stop flowing in between.  Here one CTA
// per SM stays resident for the whole step and walks a list of phases (decode_persistent.h) built by the host from the
// step's node list:
//   per layer   [norm + quantize | Q, K, V mat-muls | rope, cache write]   grid barrier
//               [attention over the cache, splits merged by the last arriver]   grid barrier
//               [quantize | attn_output mat-mul | + residual]   grid barrier
//               [norm + quantize | gate and up mat-muls | silu(gate) * up]   grid barrier
//               [quantize | ffn_down mat-mul | + residual]   grid barrier
//   at the end  [norm + quantize | output mat-mul]
// How the bytes move:
//   * warp 16 of a CTA is the PRODUCER: one lane walks the whole step's weight stream of this CTA (every phase, every
//     layer: the tile -> CTA map is static) and issues one cp.async.bulk per unit (8 consecutive 256-element groups of a
//     Q4_K row tile = 36864 bytes, or 4 of a Q6_K one = 26880) into a ring in shared memory.  It never waits for a
//     phase: it runs ahead of the consumers by the ring's depth, so the weights of the next phase are already arriving
//     while the consumers sit at a grid barrier or do attention, and HBM does not drain between the phases;
//   * warps 0-15 are the CONSUMERS, two sets of eight.  A set owns a row tile: per unit, warp j takes group j from the
//     ring (lane = row; Q6_K: two warps per group, 128 elements each), leaves its exact int32 partial dots in an
//     exchange array, and after the set's barrier the f32 accumulation chains run in ascending K exactly as the CPU
//     routes order them (Q4_K: 8x8 gemv, crates/ggml/src/repack.rs:1638-1688; Q6_K: row dot,
//     crates/ggml/src/vec_dot.rs:990-1032), so every mat-mul result is bit-identical to the stand-alone kernels';
//   * the f32 op in front of a mat-mul (RMS_NORM + MUL) and the Q8_K quantization of its input row
//     (crates/ggml/src/quants.rs:615-654) are redone by every CTA into its own shared memory: the row is a few KB in L2;
//   * attention is the fast-mode unit of flash_attn_fast.cuh, run by two groups of four consumer warps.
// Every wait (ring barriers, grid barrier) is bounded: on expiry the waiter records a code in the device's error
// word, raises the step's abort word, and every CTA leaves at its next check after waiting (bounded again) for its
// own copies in flight.  Decisions to leave are taken by one thread between two barriers, so all warps of a barrier
// group leave together.
#include <cstddef>
#include <cstdlib>

#include "act_quant.cuh"
#include "decode_persistent.h"
#include "fa_math.cuh"

namespace b200 {

namespace {

constexpr int DP_CONSUMER_WARPS = 16;
constexpr int DP_SET_WARPS = 8;
constexpr int DP_SETS = 2;
constexpr int DP_SLOTS = 2;                         // ring slots per set
constexpr int DP_SLOT_BYTES = 36864;                // 8 Q4_K chunks
constexpr int DP_THREADS = (DP_CONSUMER_WARPS + 1) * 32;
constexpr int DP_RING_BYTES = DP_SETS * DP_SLOTS * DP_SLOT_BYTES;
constexpr int DP_WORK_BYTES = 80 * 1024;            // activations + exchange (mat-mul phases) / K, V tiles (attention): aliased
constexpr int DP_XCH_WORDS = 4 * 2 * 8 * 32 + 4 * 32;   // Q6_K: [4 groups][2 halves][8 lane sums][32 rows] + [4 groups][32] scales
constexpr int DP_FA_ROWS = 4;                       // query heads per KV head one attention unit carries
constexpr int DP_FA_GROUPS = 2;                     // attention groups (of four warps) per CTA
constexpr unsigned DP_SPIN_DEFAULT = 1u << 22;      // polls with a short sleep between them: a few seconds in all
constexpr int Q4K_CHUNK = 4608, Q6K_CHUNK = 6720;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait for the phase with the given parity; gives up early when *stop becomes non-zero
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, unsigned limit, const volatile int *stop) {
    for (unsigned i = 0; i < limit; i++) {
        if (mbar_test(bar, parity)) return true;
        if (i > 8) {
            if (*stop) return false;
            __nanosleep(64);
        }
    }
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void *src_gmem, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_i32(const int *p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// profiling aid: one thread of one CTA notes where its time goes
__device__ __forceinline__ void trace_event(DpSync *sync, bool on, unsigned code) {
    if (!on) return;
    const unsigned n = sync->trace_n;
    if (n < DP_TRACE_MAX) {
        sync->trace[n] = ((unsigned long long)code << 56) | ((unsigned long long)clock64() & 0x00ffffffffffffffull);
        sync->trace_n = n + 1;
    }
}

// barrier ids: 0 = the whole CTA, 1 = the 16 consumer warps, 2 / 3 = consumer sets, 4 / 5 = attention groups
__device__ __forceinline__ void consumer_sync() { named_sync(1, DP_CONSUMER_WARPS * 32); }
struct SetSync {
    int id;
    __device__ __forceinline__ void operator()() const { named_sync(id, DP_SET_WARPS * 32); }
};
struct FaGroupSync {
    int id;
    __device__ __forceinline__ void operator()() const { named_sync(id, FF_WARPS * 32); }
};

// fixed part of the shared memory behind the ring and the work region
struct DpCtl {
    uint64_t full[DP_SETS][DP_SLOTS];
    uint64_t empty[DP_SETS][DP_SLOTS];
    double sq_part[DP_CONSUMER_WARPS];
    int abort_set[DP_SETS];      // written by a set's own warps before the set's barrier, read after it
    int abort_producer;          // the producer gave up: consumers stop waiting for its copies
    int decision;                // published by thread 0 between the two barriers of a phase boundary
    FaFastMisc fa_misc[DP_FA_GROUPS];
};

// mat-mul view of the work region
struct GemvWork {
    int8_t *aq;      // [k] quantized row
    int *bs16;       // [nb][16] 16-element sums
    int *bp;         // [nb][8] sums of 32 elements (bsums[2j] + bsums[2j+1])
    float *dx;       // [nb] block scales
    uint32_t *xch;   // [sets][2][DP_XCH_WORDS]
    float *fin;      // [sets][8][32]
};
__host__ __device__ inline size_t gemv_work_bytes(int k) {
    const size_t nb = (size_t)k / 256;
    return (size_t)k + nb * 16 * 4 + nb * 8 * 4 + (nb * 4 + 15) / 16 * 16 + (size_t)DP_SETS * 2 * DP_XCH_WORDS * 4 + (size_t)DP_SETS * 8 * 32 * 4;
}
__device__ __forceinline__ GemvWork carve_gemv(unsigned char *work, int k) {
    const size_t nb = (size_t)k / 256;
    GemvWork w;
    w.aq = (int8_t *)work;
    work += k;
    w.bs16 = (int *)work;
    work += nb * 16 * 4;
    w.bp = (int *)work;
    work += nb * 8 * 4;
    w.dx = (float *)work;
    work += (nb * 4 + 15) / 16 * 16;
    w.xch = (uint32_t *)work;
    work += (size_t)DP_SETS * 2 * DP_XCH_WORDS * 4;
    w.fin = (float *)work;
    return w;
}

__device__ __forceinline__ int units_of(int type, int nb) { return type == B200_TYPE_Q4_K ? (nb + 7) / 8 : (nb + 3) / 4; }

// job `job` of a phase, sub-tile `sub` (pair phases have two): which matrix, which of its row tiles
__device__ __forceinline__ void locate(const DpPhase &P, int job, int sub, int *m, int *tile) {
    if (P.pair) {
        *m = sub;
        *tile = job;
        return;
    }
    int t = job, i = 0;
    while (i + 1 < P.n_mat && t >= P.mat[i].n_tiles) {
        t -= P.mat[i].n_tiles;
        i++;
    }
    *m = i;
    *tile = t;
}
// first job of a set's slot in a phase; the slot then takes every (2 * grid)-th job
__device__ __forceinline__ int first_job(const DpPhase &P, int set, int cta, int grid) {
    return set * grid + (cta + grid - P.rot % grid) % grid;
}

// ---- producer ---------------------------------------------------------------------------------------------
struct ProducerState {
    int ph, job, sub, unit;      // the next unit to issue
    int n_units, gpu, chunk, nb;
    const uint8_t *tile_base;
    unsigned count;              // units issued so far
    bool fresh;                  // tile_base / n_units have to be derived
    bool done;
};

// positions st on its next unit (skipping phases without work for this slot); false when the step is exhausted
__device__ bool producer_seek(ProducerState &st, const DpPhase *phases, int n_phases, int set, int cta, int grid) {
    for (;;) {
        if (st.ph >= n_phases) {
            st.done = true;
            return false;
        }
        const DpPhase &P = phases[st.ph];
        if (P.kind != DP_GEMV) {
            st.ph++;
            st.job = -1;
            continue;
        }
        if (st.job < 0) {
            st.job = first_job(P, set, cta, grid);
            st.sub = 0;
            st.unit = 0;
            st.fresh = true;
        }
        if (st.job >= P.jobs) {
            st.ph++;
            st.job = -1;
            continue;
        }
        if (st.fresh) {
            int m, tile;
            locate(P, st.job, st.sub, &m, &tile);
            const int type = P.mat[m].type;
            st.nb = P.nb;
            st.gpu = type == B200_TYPE_Q4_K ? 8 : 4;
            st.chunk = type == B200_TYPE_Q4_K ? Q4K_CHUNK : Q6K_CHUNK;
            st.n_units = units_of(type, P.nb);
            st.tile_base = P.mat[m].tiles + (int64_t)tile * P.nb * st.chunk;
            st.fresh = false;
        }
        return true;
    }
}
__device__ __forceinline__ void producer_advance(ProducerState &st, const DpPhase *phases, int grid) {
    st.count++;
    if (++st.unit < st.n_units) return;
    st.unit = 0;
    st.fresh = true;
    const DpPhase &P = phases[st.ph];
    if (P.pair && st.sub == 0) {
        st.sub = 1;
        return;
    }
    st.sub = 0;
    st.job += DP_SETS * grid;
}

// ---- consumers: one unit of a row tile ------------------------------------------------------------------------
// Q4_K: warp j of the set takes group j of the unit; xb[(j * 3 + {0, 1, 2}) * 32 + lane] = iacc, imin, d | dmin << 16
__device__ __forceinline__ void q4k_group(const uint8_t *chunk, int lane, const int8_t *aq_g, const int *bp_g, uint32_t *xw) {
    const uint4 h = *(const uint4 *)(chunk + lane * 16);
    uint4 q[8];
#pragma unroll
    for (int c = 0; c < 8; c++) q[c] = *(const uint4 *)(chunk + 512 + c * 512 + lane * 16);
    // 6-bit scales and mins: crates/ggml/src/quants.rs:421-429 (get_scale_min_k4)
    const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
    const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu, mn_lo4 = u1 & 0x3f3f3f3fu;
    const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
    const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
    const uint4 *aq = (const uint4 *)aq_g;
    int iacc = 0;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        int dlo = 0, dhi = 0;
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const uint4 w = q[2 * g + hh];
            const uint4 alo = aq[4 * g + hh], ahi = aq[4 * g + 2 + hh];
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
        imin += (int)((m4 >> (8 * (j & 3))) & 0xff) * bp_g[j];
    }
    xw[0] = (uint32_t)iacc;
    xw[32] = (uint32_t)imin;
    xw[64] = h.x;
}

__device__ __forceinline__ uint32_t word_at(const uint4 &v, int w) { return w == 0 ? v.x : w == 1 ? v.y : w == 2 ? v.z : v.w; }
__device__ __forceinline__ int q6k_scale(const uint4 &sc, int b) { return (int)(int8_t)(word_at(sc, b >> 2) >> (8 * (b & 3))); }

// Q6_K: warps 2g and 2g + 1 of the set take elements 0..127 and 128..255 of group g.  xw[l * 32] = this half's share of
// lane sum l (half 0 also takes the -32 bias off, with the CPU's pairing of 16-element sums and scales); dw: the row's d
__device__ __forceinline__ void q6k_half(const uint8_t *chunk, int lane, int n, const int8_t *aq_g, const int *bs16_g, uint32_t *xw, uint32_t *dw) {
    uint4 ql[4], qh[2];
#pragma unroll
    for (int c = 0; c < 4; c++) ql[c] = *(const uint4 *)(chunk + (4 * n + c) * 512 + lane * 16);
#pragma unroll
    for (int c = 0; c < 2; c++) qh[c] = *(const uint4 *)(chunk + 4096 + (2 * n + c) * 512 + lane * 16);
    const uint4 sc = *(const uint4 *)(chunk + 6144 + lane * 16);
    const uint4 *aq = (const uint4 *)aq_g;
    int sumi[8];
#pragma unroll
    for (int l = 0; l < 8; l++) sumi[l] = 0;
#pragma unroll
    for (int l16 = 0; l16 < 2; l16++) {
        const uint4 A = ql[l16], B = ql[2 + l16], H = qh[l16];
        const uint4 y0 = aq[8 * n + 0 + l16], y1 = aq[8 * n + 2 + l16], y2 = aq[8 * n + 4 + l16], y3 = aq[8 * n + 6 + l16];
        const int s0 = q6k_scale(sc, 8 * n + 0 + l16), s1 = q6k_scale(sc, 8 * n + 2 + l16);
        const int s2 = q6k_scale(sc, 8 * n + 4 + l16), s3 = q6k_scale(sc, 8 * n + 6 + l16);
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const uint32_t aw = word_at(A, w), bw = word_at(B, w), hw = word_at(H, w);
            const uint32_t v0 = (aw & 0x0f0f0f0fu) | ((hw << 4) & 0x30303030u);
            const uint32_t v1 = (bw & 0x0f0f0f0fu) | ((hw << 2) & 0x30303030u);
            const uint32_t v2 = ((aw >> 4) & 0x0f0f0f0fu) | (hw & 0x30303030u);
            const uint32_t v3 = ((bw >> 4) & 0x0f0f0f0fu) | ((hw >> 2) & 0x30303030u);
            int acc = sumi[4 * l16 + w];
            acc += s0 * __dp4a((int)v0, (int)word_at(y0, w), 0);
            acc += s1 * __dp4a((int)v1, (int)word_at(y1, w), 0);
            acc += s2 * __dp4a((int)v2, (int)word_at(y2, w), 0);
            acc += s3 * __dp4a((int)v3, (int)word_at(y3, w), 0);
            sumi[4 * l16 + w] = acc;
        }
    }
#pragma unroll
    for (int l = 0; l < 8; l++) {
        int v = sumi[l];
        if (n == 0) v -= (bs16_g[2 * l] * q6k_scale(sc, 2 * l) + bs16_g[2 * l + 1] * q6k_scale(sc, 2 * l + 1)) * 32;
        xw[l * 32] = (uint32_t)v;
    }
    if (n == 0) *dw = *(const uint16_t *)(chunk + 6656 + lane * 2);
}

// the row this CTA multiplies by, quantized into shared memory (every consumer warp)
constexpr int DP_PRO_BLOCKS = 4;   // 256-element blocks a warp holds in registers at a time
__device__ void dp_prologue(const DpPhase &P, const GemvWork &W, DpCtl *ctl, int warp, int lane, bool writer) {
    const int nb = P.nb;
    // Every warp loads all its blocks (b = warp, warp + 16, ...) before it uses any: the loads are independent, so a
    // warp pays one trip to L2 for them, not one per block.  A NORM row is at most DP_PRO_BLOCKS * 16 blocks (checked
    // by the host), so its values stay in registers between the sum of squares and the quantization.
    for (int base = 0; base < nb; base += DP_PRO_BLOCKS * DP_CONSUMER_WARPS) {
        float v[DP_PRO_BLOCKS][8], ws[DP_PRO_BLOCKS][8];
#pragma unroll
        for (int i = 0; i < DP_PRO_BLOCKS; i++) {
            const int b = base + warp + i * DP_CONSUMER_WARPS;
            if (b < nb) {
                const int64_t e0 = (int64_t)b * 256 + 8 * lane;
                const float4 a0 = __ldcg((const float4 *)(P.x + e0)), a1 = __ldcg((const float4 *)(P.x + e0 + 4));
                v[i][0] = a0.x; v[i][1] = a0.y; v[i][2] = a0.z; v[i][3] = a0.w; v[i][4] = a1.x; v[i][5] = a1.y; v[i][6] = a1.z; v[i][7] = a1.w;
                if (P.prologue == DP_PRO_NORM) {
                    const float4 w0 = __ldg((const float4 *)(P.norm_w + e0)), w1 = __ldg((const float4 *)(P.norm_w + e0 + 4));
                    ws[i][0] = w0.x; ws[i][1] = w0.y; ws[i][2] = w0.z; ws[i][3] = w0.w; ws[i][4] = w1.x; ws[i][5] = w1.y; ws[i][6] = w1.z; ws[i][7] = w1.w;
                }
            }
        }
        float rms_scale = 1.0f;
        if (P.prologue == DP_PRO_NORM) {
            // the row's squares summed in f64: crates/ggml/src/compute.rs:2634-2683
            double sum = 0.0;
#pragma unroll
            for (int i = 0; i < DP_PRO_BLOCKS; i++)
                if (base + warp + i * DP_CONSUMER_WARPS < nb) {
#pragma unroll
                    for (int j = 0; j < 8; j++) sum += (double)__fmul_rn(v[i][j], v[i][j]);
                }
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) ctl->sq_part[warp] = sum;
            consumer_sync();
            double total = 0.0;
            for (int i = 0; i < DP_CONSUMER_WARPS; i++) total += ctl->sq_part[i];
            const float mean = __double2float_rn(total / (double)(nb * 256));
            rms_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, P.eps)));
        }
#pragma unroll
        for (int i = 0; i < DP_PRO_BLOCKS; i++) {
            const int b = base + warp + i * DP_CONSUMER_WARPS;
            if (b >= nb) continue;
            const int64_t e0 = (int64_t)b * 256 + 8 * lane;
            if (P.prologue == DP_PRO_NORM) {
                float nv[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    nv[j] = __fmul_rn(v[i][j], rms_scale);
                    v[i][j] = __fmul_rn(nv[j], ws[i][j]);
                }
                if (writer) {
                    if (P.y) {
                        *(float4 *)(P.y + e0) = make_float4(nv[0], nv[1], nv[2], nv[3]);
                        *(float4 *)(P.y + e0 + 4) = make_float4(nv[4], nv[5], nv[6], nv[7]);
                    }
                    if (P.y_mul) {
                        *(float4 *)(P.y_mul + e0) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
                        *(float4 *)(P.y_mul + e0 + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
                    }
                }
            }
            // quantize_row_q8_K on the block the warp holds (lane l: elements 8 l .. 8 l + 7)
            uint2 packed;
            float d;
            int s8;
            q8_K_block_regs(v[i], &packed, &d, &s8);
            *(uint2 *)(W.aq + e0) = packed;
            const int s16 = s8 + __shfl_xor_sync(0xffffffffu, s8, 1);
            const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 2);
            if ((lane & 1) == 0) W.bs16[b * 16 + (lane >> 1)] = s16;
            if ((lane & 3) == 0) W.bp[b * 8 + (lane >> 2)] = s32;
            if (lane == 0) W.dx[b] = d;
        }
    }
    consumer_sync();
}
size_t dp_norm_max_blocks() { return (size_t)DP_PRO_BLOCKS * DP_CONSUMER_WARPS; }

// what warp 0 of a set does with a finished row tile (lane = row)
__device__ __forceinline__ void dp_epilogue(const DpPhase &P, const DpMat &M, int tile, int lane, float v, int *err) {
    const int64_t row = (int64_t)tile * TILE_ROWS + lane;
    switch (M.epi) {
        case DP_EPI_STORE: M.dst[row] = v; break;
        case DP_EPI_ADD:
            M.dst[row] = v;
            P.sum[row] = __fadd_rn(v, __ldcg(P.addend + row));
            break;
        case DP_EPI_ROPE:
        case DP_EPI_ROPE_CACHE: {
            // crates/ggml/src/compute.rs:3663-3677 rotate_pairs_f32, adjacent channels (mode NORMAL): the pair sits in two
            // neighbouring lanes
            if (M.dst_raw) M.dst_raw[row] = v;
            const float other = __shfl_xor_sync(0xffffffffu, v, 1);
            const int64_t tr = (int64_t)__ldg(P.pos);
            const int e = (int)(row % P.head_dim), i0 = e & ~1;
            float out = v;
            bool ok = true;
            if (i0 < P.n_dims) {
                if (tr < 0 || tr >= P.rope_rows) {
                    if (lane == 0) atomicExch(err, 3);
                    ok = false;
                } else {
                    const float c = __ldg(P.rope_table + tr * P.head_dim + i0), s = __ldg(P.rope_table + tr * P.head_dim + i0 + 1);
                    const float x0 = (e & 1) ? other : v, x1 = (e & 1) ? v : other;
                    out = (e & 1) ? __fmaf_rn(x0, s, __fmul_rn(x1, c)) : __fmaf_rn(x0, c, -__fmul_rn(x1, s));
                }
            }
            if (ok) {
                M.dst[row] = out;
                if (M.epi == DP_EPI_ROPE_CACHE) {
                    const int64_t cell = *P.cell;
                    if (cell < 0 || cell >= P.cache_rows) {
                        if (lane == 0) atomicExch(err, 2);
                    } else {
                        M.cache[cell * P.cache_stride + row] = __float2half_rn(out);
                    }
                }
            }
            break;
        }
        case DP_EPI_CACHE: {
            M.dst[row] = v;
            const int64_t cell = *P.cell;
            if (cell < 0 || cell >= P.cache_rows) {
                if (lane == 0) atomicExch(err, 2);
            } else {
                M.cache[cell * P.cache_stride + row] = __float2half_rn(v);
            }
            break;
        }
        default: break;
    }
}

__global__ void __launch_bounds__(DP_THREADS, 1)
decode_persistent_kernel(const DpPhase *__restrict__ phases, int n_phases, DpSync *sync, int *err, unsigned spin_limit, int skip_cta,
                         int skip_barrier, int profile, int pf_ahead) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char *ring = smem_raw;
    unsigned char *work = smem_raw + DP_RING_BYTES;
    DpCtl *ctl = (DpCtl *)(work + DP_WORK_BYTES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, grid = gridDim.x;

    if (tid == 0) {
        for (int s = 0; s < DP_SETS; s++)
            for (int i = 0; i < DP_SLOTS; i++) {
                mbar_init(&ctl->full[s][i], 1);
                mbar_init(&ctl->empty[s][i], 1);
            }
        ctl->abort_set[0] = ctl->abort_set[1] = 0;
        ctl->abort_producer = 0;
        ctl->decision = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const volatile int *stop_p = (const volatile int *)&ctl->abort_producer;

    // what the producer lane has in flight, for the wind-down
    unsigned issued[DP_SETS] = {0, 0};
    if (warp == DP_CONSUMER_WARPS) {
        // ================= producer: the weights do not depend on anything the step computes =================
        if (lane == 0) {
            // st: the next unit to copy into the ring; pf: the next unit to ask L2 for, pf_ahead units further down the
            // same stream, so that HBM keeps working while the ring is full (consumers at a grid barrier or in attention)
            ProducerState st[DP_SETS], pf[DP_SETS];
            for (int s = 0; s < DP_SETS; s++) {
                st[s].ph = 0; st[s].job = -1; st[s].sub = 0; st[s].unit = 0; st[s].count = 0; st[s].fresh = true; st[s].done = false;
                producer_seek(st[s], phases, n_phases, s, cta, grid);
                pf[s] = st[s];
            }
            unsigned idle = 0;
            while (!(st[0].done && st[1].done)) {
                bool progressed = false;
#pragma unroll
                for (int s = 0; s < DP_SETS; s++) {
                    if (st[s].done) continue;
                    const unsigned c = st[s].count;
                    const int slot = (int)(c % DP_SLOTS);
                    // the slot's previous use (unit c - DP_SLOTS) must have been released
                    if (c >= DP_SLOTS && !mbar_test(&ctl->empty[s][slot], ((c / DP_SLOTS) & 1u) ^ 1u)) continue;
                    const int g0 = st[s].unit * st[s].gpu;
                    const int ng = st[s].nb - g0 < st[s].gpu ? st[s].nb - g0 : st[s].gpu;
                    const unsigned bytes = (unsigned)(ng * st[s].chunk);
                    mbar_expect_tx(&ctl->full[s][slot], bytes);
                    bulk_load(ring + (size_t)(s * DP_SLOTS + slot) * DP_SLOT_BYTES, st[s].tile_base + (int64_t)g0 * st[s].chunk, bytes,
                              &ctl->full[s][slot]);
                    issued[s] = c + 1;
                    producer_advance(st[s], phases, grid);
                    producer_seek(st[s], phases, n_phases, s, cta, grid);
                    progressed = true;
                }
                if (pf_ahead > 0) {
#pragma unroll
                    for (int s = 0; s < DP_SETS; s++) {
                        int budget = 2;   // a couple per turn: the ring comes first
                        while (!pf[s].done && pf[s].count < st[s].count + (unsigned)pf_ahead && budget > 0) {
                            if (pf[s].count >= st[s].count) {
                                const int g0 = pf[s].unit * pf[s].gpu;
                                const int ng = pf[s].nb - g0 < pf[s].gpu ? pf[s].nb - g0 : pf[s].gpu;
                                bulk_prefetch_l2(pf[s].tile_base + (int64_t)g0 * pf[s].chunk, (unsigned)(ng * pf[s].chunk));
                                budget--;
                                progressed = true;
                            }
                            producer_advance(pf[s], phases, grid);
                            producer_seek(pf[s], phases, n_phases, s, cta, grid);
                        }
                    }
                }
                if (progressed) {
                    idle = 0;
                    continue;
                }
                if (++idle > spin_limit) {
                    atomicExch(err, 6);
                    atomicExch(&sync->abort, 1);
                    *(volatile int *)&ctl->abort_producer = 1;
                    break;
                }
                if (idle > 8) {
                    if (ctl->abort_set[0] | ctl->abort_set[1] | (*(volatile int *)&ctl->decision == 0)) break;
                    if ((idle & 63) == 0 && ld_relaxed_i32(&sync->abort)) break;
                    __nanosleep(64);
                }
            }
        }
    } else {
        // ================= consumers =================
        const int set = warp / DP_SET_WARPS, wj = warp % DP_SET_WARPS;
        const SetSync set_sync{2 + set};
        if (cta == 0 && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            sync->t_phase[0] = t;
        }
        const bool tr = profile > 1 && cta == profile - 2 && tid == 0;   // B200_DECODE_PROFILE = 2 + c: trace CTA c
        unsigned count = 0;        // units this set has consumed
        unsigned barrier_no = 0;   // grid barriers passed
        bool alive = true;
        for (int ph = 0; ph < n_phases && alive; ph++) {
            const DpPhase &P = phases[ph];
            if (P.kind == DP_GEMV) {
                const GemvWork W = carve_gemv(work, P.k);
                const int j0 = first_job(P, 0, cta, grid);   // set 0's first job: the CTA has work in this phase iff it exists
                if (j0 < P.jobs) {
                    trace_event(sync, tr, 1);
                    dp_prologue(P, W, ctl, warp, lane, j0 == 0);
                    trace_event(sync, tr, 2);
                    uint32_t *xch = W.xch + (size_t)set * 2 * DP_XCH_WORDS;
                    float *fin = W.fin + (size_t)set * 8 * 32;
                    bool set_alive = true;
                    const int nsub = P.pair ? 2 : 1;
                    for (int job = first_job(P, set, cta, grid); job < P.jobs && set_alive; job += DP_SETS * grid) {
                        float keep = 0.0f;   // pair: the first sub-tile's outputs (warp 0 of the set, lane = row)
                        for (int sub = 0; sub < nsub && set_alive; sub++) {
                            int m, tile;
                            locate(P, job, sub, &m, &tile);
                            const DpMat &M = P.mat[m];
                            const bool q4 = M.type == B200_TYPE_Q4_K;
                            const int gpu = q4 ? 8 : 4, chunk = q4 ? Q4K_CHUNK : Q6K_CHUNK;
                            const int n_units = units_of(M.type, P.nb);
                            float acc0 = 0.0f, acc1 = 0.0f;   // Q4_K (warp 0): sumf, summin; Q6_K (warp l): lane accumulator l
                            for (int u = 0; u < n_units; u++, count++) {
                                const int slot = (int)(count % DP_SLOTS);
                                int ok = 1;
                                if (lane == 0) ok = mbar_wait(&ctl->full[set][slot], (count / DP_SLOTS) & 1u, spin_limit, stop_p) ? 1 : 0;
                                ok = __shfl_sync(0xffffffffu, ok, 0);
                                trace_event(sync, tr, 3);
                                const int g0 = u * gpu;
                                const int ng = P.nb - g0 < gpu ? P.nb - g0 : gpu;
                                uint32_t *xb = xch + (size_t)(count & 1u) * DP_XCH_WORDS;
                                if (!ok) {
                                    if (lane == 0) {
                                        atomicExch(err, 7);
                                        *(volatile int *)&ctl->abort_set[set] = 1;
                                    }
                                } else {
                                    const uint8_t *sl = ring + (size_t)(set * DP_SLOTS + slot) * DP_SLOT_BYTES;
                                    if (q4) {
                                        if (wj < ng) {
                                            const int b = g0 + wj;
                                            q4k_group(sl + (size_t)wj * Q4K_CHUNK, lane, W.aq + (size_t)b * 256, W.bp + b * 8, xb + wj * 3 * 32 + lane);
                                        }
                                    } else {
                                        const int g = wj >> 1, n = wj & 1;
                                        if (g < ng) {
                                            const int b = g0 + g;
                                            q6k_half(sl + (size_t)g * Q6K_CHUNK, lane, n, W.aq + (size_t)b * 256, W.bs16 + b * 16,
                                                     xb + ((g * 2 + n) * 8) * 32 + lane, xb + 4 * 2 * 8 * 32 + g * 32 + lane);
                                        }
                                    }
                                }
                                trace_event(sync, tr, 4);
                                set_sync();
                                trace_event(sync, tr, 5);
                                if (*(volatile int *)&ctl->abort_set[set]) {
                                    set_alive = false;
                                    break;
                                }
                                if (wj == 0 && lane == 0) mbar_arrive(&ctl->empty[set][slot]);   // everyone of the set has read the slot
                                // the unit's share of the chains, ascending K
                                if (q4) {
                                    if (wj == 0) {
                                        for (int g = 0; g < ng; g++) {
                                            const uint32_t *xe = xb + g * 3 * 32 + lane;
                                            const int vi = (int)xe[0], vm = (int)xe[32];
                                            const uint32_t hd = xe[64];
                                            const float d = f16_bits_to_f32((uint16_t)(hd & 0xffffu)), dmin = f16_bits_to_f32((uint16_t)(hd >> 16));
                                            const float da = W.dx[g0 + g];
                                            acc0 = __fmaf_rn((float)vi, __fmul_rn(d, da), acc0);
                                            acc1 = __fmaf_rn((float)vm, __fmul_rn(dmin, da), acc1);
                                        }
                                    }
                                } else {
                                    for (int g = 0; g < ng; g++) {
                                        const int si = (int)xb[((g * 2 + 0) * 8 + wj) * 32 + lane] + (int)xb[((g * 2 + 1) * 8 + wj) * 32 + lane];
                                        const float dw = f16_bits_to_f32((uint16_t)xb[4 * 2 * 8 * 32 + g * 32 + lane]);
                                        acc0 = __fmaf_rn(__fmul_rn(W.dx[g0 + g], dw), (float)si, acc0);
                                    }
                                }
                            }
                            if (!set_alive) break;
                            trace_event(sync, tr, 6);
                            float v = 0.0f;
                            if (q4) {
                                v = __fsub_rn(acc0, acc1);
                            } else {
                                // hsum8 of the eight lane accumulators: crates/ggml/src/vec_dot.rs:564-572
                                fin[wj * 32 + lane] = acc0;
                                set_sync();
                                if (wj == 0) {
                                    const float *a = fin + lane;
                                    const float r0 = __fadd_rn(a[4 * 32], a[0]), r1 = __fadd_rn(a[5 * 32], a[32]);
                                    const float r2 = __fadd_rn(a[6 * 32], a[2 * 32]), r3 = __fadd_rn(a[7 * 32], a[3 * 32]);
                                    v = __fadd_rn(__fadd_rn(r0, r2), __fadd_rn(r1, r3));
                                }
                            }
                            if (wj == 0) {
                                if (P.pair) {
                                    const int64_t row = (int64_t)tile * TILE_ROWS + lane;
                                    if (sub == 0) {
                                        keep = v;
                                        if (P.raw0) P.raw0[row] = v;
                                    } else {
                                        // SILU then MUL: crates/ggml/src/simd_x86.rs:1012-1054, crates/llama/src/graph_arch.rs:1150-1151
                                        if (P.raw1) P.raw1[row] = v;
                                        const float e = (int)row < P.wide_end ? v_expf(__fsub_rn(0.0f, keep)) : libm_expf(-keep);
                                        const float sv = __fdiv_rn(keep, __fadd_rn(1.0f, e));
                                        if (P.silu_out) P.silu_out[row] = sv;
                                        P.h_out[row] = __fmul_rn(sv, v);
                                    }
                                } else {
                                    dp_epilogue(P, M, tile, lane, v, err);
                                }
                            }
                            trace_event(sync, tr, 7);
                        }
                    }
                }
            } else {
                // ---- attention: (KV head, split) units over two groups of four warps
                if (warp < DP_FA_GROUPS * FF_WARPS) {
                    const int fg = warp / FF_WARPS;
                    const FaGroupSync fsync{4 + fg};
                    unsigned char *fsm = work + (size_t)fg * fa_fast_smem_bytes<128, DP_FA_ROWS, 2>();
                    if ((tid & (FF_WARPS * 32 - 1)) == 0) ctl->fa_misc[fg].vis_list = nullptr;
                    const int units = P.fd.H_kv * P.fd.n_splits;
                    for (int u = fg * grid + cta; u < units; u += DP_FA_GROUPS * grid) {
                        const int hk = u / P.fd.n_splits, split = u - hk * P.fd.n_splits;
                        fsync();   // the group's shared memory is free again
                        fa_fast_unit<128, DP_FA_ROWS, 2>(P.fa, P.fd, P.scale_log2, P.partial, P.counters, split, hk, 0, 1, tid & (FF_WARPS * 32 - 1), fsm,
                                                      &ctl->fa_misc[fg], fsync);
                    }
                }
            }
            trace_event(sync, tr, 8);
            if (ph + 1 == n_phases) break;
            // ---- phase boundary: grid barrier.  Thread 0 decides between two barriers of the consumers whether the CTA goes on.
            consumer_sync();
            if (tid == 0) {
                bool go = !(ctl->abort_set[0] | ctl->abort_set[1] | ctl->abort_producer);
                if (!go) atomicExch(&sync->abort, 1);
                __threadfence();
                if (profile && barrier_no < DP_MAX_TIMED) {
                    unsigned long long t;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                    atomicMin(&sync->t_first[barrier_no], t);
                    atomicMax(&sync->t_last[barrier_no], t);
                }
                if (!(cta == skip_cta && (int)barrier_no == skip_barrier)) atomicAdd(&sync->arrived, 1u);
                const unsigned target = (barrier_no + 1u) * (unsigned)grid;
                bool reached = false;
                for (unsigned i = 0; i < spin_limit; i++) {
                    if (ld_acquire_u32(&sync->arrived) >= target) {
                        reached = true;
                        break;
                    }
                    if (ld_relaxed_i32(&sync->abort)) break;
                    if (i > 16) __nanosleep(i > 1024 ? 256 : 32);
                }
                if (!reached) {
                    if (!ld_relaxed_i32(&sync->abort)) atomicExch(err, 5);   // the wait ran out by itself
                    atomicExch(&sync->abort, 1);
                    go = false;
                }
                if (ld_relaxed_i32(&sync->abort)) go = false;
                __threadfence();
                *(volatile int *)&ctl->decision = go ? 1 : 0;
                if (cta == 0 && barrier_no + 1 < DP_MAX_TIMED) {
                    unsigned long long t;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                    sync->t_phase[barrier_no + 1] = t;
                }
            }
            consumer_sync();
            trace_event(sync, tr, 9);
            if (*(volatile int *)&ctl->decision == 0) alive = false;
            barrier_no++;
        }
        // a CTA whose set gave up in the last phase still tells the others
        if (alive && tid == 0 && (ctl->abort_set[0] | ctl->abort_set[1])) atomicExch(&sync->abort, 1);
        if (tid == 0 && !alive) *(volatile int *)&ctl->decision = 0;
    }
    // wind-down: every bulk copy this CTA issued must have landed before its shared memory is released.  On the normal
    // path the consumers have waited for each of them; after an abort the producer lane waits (bounded) for the last
    // copy it started on every slot.
    __syncthreads();
    if (warp == DP_CONSUMER_WARPS && lane == 0) {
        const bool aborted = ctl->abort_set[0] | ctl->abort_set[1] | ctl->abort_producer | (*(volatile int *)&ctl->decision == 0);
        if (aborted) {
            int never = 0;
            for (int s = 0; s < DP_SETS; s++)
                for (unsigned back = 0; back < DP_SLOTS && back < issued[s]; back++) {
                    const unsigned c = issued[s] - 1 - back;
                    mbar_wait(&ctl->full[s][c % DP_SLOTS], (c / DP_SLOTS) & 1u, spin_limit < 65536u ? 65536u : spin_limit, &never);
                }
        }
    }
}

int g_debug_spin = 0, g_debug_skip_cta = -1, g_debug_skip_barrier = -1;
unsigned long long g_launches = 0;
DpSync *g_last_sync = nullptr;

}  // namespace

size_t decode_persistent_attn_partial_bytes(int n_head_kv, int n_splits, int head_dim) {
    return (size_t)n_head_kv * n_splits * DP_FA_ROWS * (head_dim + 4) * sizeof(float);
}

void decode_persistent_debug(int spin_limit, int skip_cta, int skip_barrier) {
    g_debug_spin = spin_limit > 0 ? spin_limit : 0;
    g_debug_skip_cta = skip_cta;
    g_debug_skip_barrier = skip_barrier;
}

unsigned long long decode_persistent_launches() { return g_launches; }
// nanosecond stamps of the last launch's phase boundaries (CTA 0), after the stream has drained; returns how many were copied
int decode_persistent_times(unsigned long long *out, int n) {
    if (!g_last_sync || n <= 0) return 0;
    if (n > 3 * DP_MAX_TIMED + DP_TRACE_MAX + 1) n = 3 * DP_MAX_TIMED + DP_TRACE_MAX + 1;   // t_phase, t_first, t_last, trace, trace_n
    if (cudaMemcpy(out, g_last_sync->t_phase, (size_t)n * sizeof(unsigned long long), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}
size_t decode_persistent_work_bytes(int k) { return gemv_work_bytes(k); }
size_t decode_persistent_work_limit() { return DP_WORK_BYTES; }
int decode_persistent_norm_max_k() { return (int)dp_norm_max_blocks() * 256; }

int launch_decode_persistent(const DpPhase *dev_phases, int n_phases, DpSync *dev_sync, cudaStream_t s) {
    static_assert(DP_FA_GROUPS * fa_fast_smem_bytes<128, DP_FA_ROWS, 2>() <= DP_WORK_BYTES, "attention tiles do not fit the work region");
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "decode step: device index %d out of range", dev);
    static int sm_count[64] = {0};
    static bool attr_done[64] = {false};
    const size_t smem = (size_t)DP_RING_BYTES + DP_WORK_BYTES + sizeof(DpCtl);
    if (!attr_done[dev]) {
        cudaDeviceProp p;
        B200_CUDA(cudaGetDeviceProperties(&p, dev));
        B200_REQUIRE(p.cooperativeLaunch != 0, "decode step: the device has no cooperative launch");
        B200_REQUIRE(smem <= (size_t)p.sharedMemPerBlockOptin, "decode step: %zu bytes of shared memory per CTA exceed the device's %zu", smem,
                     (size_t)p.sharedMemPerBlockOptin);
        sm_count[dev] = p.multiProcessorCount;
        B200_CUDA(cudaFuncSetAttribute(decode_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    // B200_DECODE_L2_AHEAD: how many ring units ahead of its copies a CTA's producer asks L2 for (per consumer set)
    static int pf_ahead = -1;
    if (pf_ahead < 0) {
        const char *e = getenv("B200_DECODE_L2_AHEAD");
        pf_ahead = e ? atoi(e) : 6;
        if (pf_ahead < 0) pf_ahead = 0;
        if (pf_ahead > 64) pf_ahead = 64;
    }
    static int profile = -1;
    if (profile < 0) {
        const char *e = getenv("B200_DECODE_PROFILE");
        profile = e ? atoi(e) : 0;
    }
    B200_CUDA(cudaMemsetAsync(dev_sync, 0, offsetof(DpSync, t_first), s));
    if (profile) {
        B200_CUDA(cudaMemsetAsync(dev_sync->t_first, 0xff, sizeof(dev_sync->t_first), s));
        B200_CUDA(cudaMemsetAsync(dev_sync->t_last, 0, sizeof(dev_sync->t_last), s));
        B200_CUDA(cudaMemsetAsync(&dev_sync->trace_n, 0, sizeof(unsigned), s));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count[dev]);
    cfg.blockDim = dim3(DP_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident at once, or the launch fails: the grid barrier needs it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, decode_persistent_kernel, dev_phases, n_phases, dev_sync, err,
                                 g_debug_spin > 0 ? (unsigned)g_debug_spin : DP_SPIN_DEFAULT, g_debug_skip_cta, g_debug_skip_barrier, profile, pf_ahead));
    g_launches++;
    g_last_sync = dev_sync;
    return B200_STATUS_SUCCESS;
}

}  // namespace b200
