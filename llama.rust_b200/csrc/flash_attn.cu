// FLASH_ATTN_EXT over an F16 KV cache, decode-shaped (fewer than 64 query rows).
//
// "Faithful" mode reproduces the arithmetic of the CPU path exactly:
//   * scores: the f16 dot of crates/ggml/src/vec_dot.rs:1982-2019 (q rounded to
//     f16, 4 x 16 f32 FMA lanes over 64-element chunks, fixed fold and tree);
//   * online softmax per row with the running maximum, the F16-V accumulator
//     kept in f16 with one rounding per scale and per multiply-add, S updated
//     with one FMA (crates/ggml/src/flash_attn.rs:482-694);
//   * split-KV (one query row, n_kv >= 512): n_chunks independent chunk scans
//     merged in chunk order (flash_attn.rs:744-859); the result depends on
//     n_chunks exactly as the CPU result depends on its thread count;
//   * expf: the table-driven double-precision algorithm the host libm uses, so
//     ms / vs are the same bits (checked exhaustively against expf on the host).
// Three kernels: scores (parallel over positions), rows (one CTA per (row,
// chunk): prefix-max scan per 128-position tile, then the sequential f16
// accumulation with one thread per value element), merge.
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "fa_math.cuh"

namespace b200 {

__device__ __forceinline__ float r16(float v) { return __half2float(__float2half_rn(v)); }
// r16 for the long dependent chains: in the normal f16 range [2^-14, 65520) rounding to nearest even at
// bit 13 of the f32 pattern is three integer operations; everything else takes the conversion pair
__device__ __forceinline__ float r16_fast(float v) {
    const uint32_t b = __float_as_uint(v);
    if (((b & 0x7fffffffu) - 0x38800000u) < (0x477ff000u - 0x38800000u))
        return __uint_as_float((b + 0x0fffu + ((b >> 13) & 1u)) & 0xffffe000u);
    return r16(v);
}

struct FaDims {
    int dk, dv, T, H, H_kv;
    int64_t n_kv;
    int n_chunks;
    int64_t chunk;      // positions per chunk
};

// ---------------------------------------------------------------------------
// scores[(t*H + h)*n_kv + p] = dot(k[p], f16(q)) * kq_scale (softcap) + slope*mask,
// or -inf for a masked position (the CPU skips those entirely).
// One thread per position; the K row sits in registers and serves the
// H/H_kv heads of its group and all T query rows.
// ---------------------------------------------------------------------------
template <int DK>
__global__ void __launch_bounds__(128)
fa_scores_kernel(b200_flash_attn_args a, FaDims d, float kq_scale, float *__restrict__ scores) {
    extern __shared__ float q_s[];   // [rows in batch][DK], q rounded to f16
    const int group = d.H / d.H_kv;
    const int hkv = blockIdx.y;
    const int64_t p = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const bool live = p < d.n_kv;
    __half2 kr[DK / 2];
    if (live) {
        const uint4 *src = (const uint4 *)((const uint8_t *)a.k + p * a.k_nb1 + (int64_t)hkv * a.k_nb2);
#pragma unroll
        for (int i = 0; i < DK / 8; i++) {
            const uint4 v = src[i];
            kr[4 * i + 0] = *(const __half2 *)&v.x;
            kr[4 * i + 1] = *(const __half2 *)&v.y;
            kr[4 * i + 2] = *(const __half2 *)&v.z;
            kr[4 * i + 3] = *(const __half2 *)&v.w;
        }
    }
    const int rows_total = d.T * group;           // row = t * group + g
    constexpr int RB = 8;
    for (int r0 = 0; r0 < rows_total; r0 += RB) {
        const int nr = rows_total - r0 < RB ? rows_total - r0 : RB;
        __syncthreads();
        for (int i = threadIdx.x; i < nr * DK; i += 128) {
            const int r = r0 + i / DK, e = i % DK;
            const int t = r / group, h = hkv * group + r % group;
            const float *q = (const float *)((const uint8_t *)a.q + (int64_t)t * a.q_nb1 + (int64_t)h * a.q_nb2);
            q_s[i] = r16(q[e]);
        }
        __syncthreads();
        if (!live) continue;
        for (int rr = 0; rr < nr; rr++) {
            const int r = r0 + rr;
            const int t = r / group, h = hkv * group + r % group;
            const float *q = q_s + rr * DK;
            // a position the mask hides scores -inf whatever the dot is (the CPU skips it before the dot too)
            if (a.mask && __half2float(((const __half *)((const uint8_t *)a.mask + (int64_t)t * a.mask_nb1))[p]) == -INFINITY) {
                scores[((int64_t)t * d.H + h) * d.n_kv + p] = -INFINITY;
                continue;
            }
            float val[16];
#pragma unroll
            for (int l = 0; l < 16; l++) {
                float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                for (int c = 0; c < DK / 64; c++) {
                    const int e = 64 * c + l;
                    const float k0 = (e & 1) ? __high2float(kr[e >> 1]) : __low2float(kr[e >> 1]);
                    const float k1 = ((e + 16) & 1) ? __high2float(kr[(e + 16) >> 1]) : __low2float(kr[(e + 16) >> 1]);
                    const float k2 = ((e + 32) & 1) ? __high2float(kr[(e + 32) >> 1]) : __low2float(kr[(e + 32) >> 1]);
                    const float k3 = ((e + 48) & 1) ? __high2float(kr[(e + 48) >> 1]) : __low2float(kr[(e + 48) >> 1]);
                    s0 = __fmaf_rn(q[e], k0, s0);
                    s1 = __fmaf_rn(q[e + 16], k1, s1);
                    s2 = __fmaf_rn(q[e + 32], k2, s2);
                    s3 = __fmaf_rn(q[e + 48], k3, s3);
                }
                val[l] = __fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3));
            }
#pragma unroll
            for (int half = 8; half >= 1; half >>= 1)
#pragma unroll
                for (int i = 0; i < half; i++) val[i] = __fadd_rn(val[i], val[i + half]);
            float s = __fmul_rn(val[0], kq_scale);
            if (a.logit_softcap != 0.0f) s = __fmul_rn(a.logit_softcap, tanhf(s));
            if (a.mask) {
                const __half mh = ((const __half *)((const uint8_t *)a.mask + (int64_t)t * a.mask_nb1))[p];
                float slope = 1.0f;
                if (a.max_bias > 0.0f) {
                    // ALiBi slope of head h: crates/ggml/src/flash_attn.rs:356-370
                    const unsigned nl2 = 1u << (31 - __clz((unsigned)d.H));
                    const float m0 = powf(2.0f, -a.max_bias / (float)nl2);
                    const float m1 = powf(2.0f, -(a.max_bias / 2.0f) / (float)nl2);
                    const float base = (unsigned)h < nl2 ? m0 : m1;
                    const int ex = (unsigned)h < nl2 ? h + 1 : 2 * (h - (int)nl2) + 1;
                    float acc = 1.0f, b = base;   // powi by repeated squaring
                    for (int e2 = ex; e2 > 0; e2 >>= 1) {
                        if (e2 & 1) acc = __fmul_rn(acc, b);
                        b = __fmul_rn(b, b);
                    }
                    slope = acc;
                }
                const float mv = __fmul_rn(slope, __half2float(mh));
                s = (mv == -INFINITY) ? -INFINITY : __fadd_rn(s, mv);
            }
            scores[((int64_t)t * d.H + h) * d.n_kv + p] = s;
        }
    }
}

// ---------------------------------------------------------------------------
// rows: grid (chunk, h, t), block = 128 value threads + 1 warp for the S chain.
// Writes per (row, chunk): M, S, and the unnormalized accumulator (f32 view).
// ---------------------------------------------------------------------------
constexpr int FA_TILE = 128;

__global__ void __launch_bounds__(160)
fa_rows_kernel(b200_flash_attn_args a, FaDims d, const float *__restrict__ scores, float *__restrict__ partials) {
    extern __shared__ __align__(16) unsigned char fsm[];
    __half *v_s = (__half *)fsm;                                  // [FA_TILE][dv]
    float *ms_s = (float *)(fsm + (size_t)FA_TILE * d.dv * 2);    // [FA_TILE]
    float *vs_s = ms_s + FA_TILE;
    float *wmax = vs_s + FA_TILE;                                 // [4] warp maxima
    __shared__ float carry_M;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
    const int hkv = h / (d.H / d.H_kv);
    const int64_t ic0 = (int64_t)c * d.chunk;
    const int64_t ic1 = ic0 + d.chunk < d.n_kv ? ic0 + d.chunk : d.n_kv;
    const int64_t row = (int64_t)t * d.H + h;
    float *part = partials + (row * d.n_chunks + c) * (2 + d.dv);
    if (ic0 >= d.n_kv) {   // out-of-range chunk: M = -inf, S = 0 (flash_attn.rs:757-764)
        if (tid == 0) { part[0] = -INFINITY; part[1] = 0.0f; }
        return;
    }
    const float *srow = scores + row * d.n_kv;
    const uint8_t *vbase = (const uint8_t *)a.v + (int64_t)hkv * a.v_nb2;
    if (tid == 0) carry_M = -INFINITY;
    float x = 0.0f;      // value threads: accumulator element d = tid (f16-representable)
    float S = 0.0f;      // S-chain lane
    const bool is_val = tid < d.dv;
    const bool is_s = tid == 128;
    __syncthreads();
    for (int64_t p0 = ic0; p0 < ic1; p0 += FA_TILE) {
        const int np = ic1 - p0 < FA_TILE ? (int)(ic1 - p0) : FA_TILE;
        float s = -INFINITY;
        if (tid < FA_TILE && tid < np) s = srow[p0 + tid];
        // a tile without a live position (another sequence's cells in a shared cache) changes nothing: skip it whole
        if (!__syncthreads_or(s != -INFINITY)) continue;
        // stage the V tile: np rows of dv halves, 16 bytes per load
        const int chunks_per_row = d.dv / 8;
        for (int i = tid; i < np * chunks_per_row; i += blockDim.x) {
            const int pr = i / chunks_per_row, cc = i % chunks_per_row;
            const uint4 v = *(const uint4 *)(vbase + (p0 + pr) * a.v_nb1 + cc * 16);
            *(uint4 *)(v_s + pr * d.dv + cc * 8) = v;
        }
        // exclusive prefix maximum of the tile's scores (threads 0..127 = positions)
        float incl = s;
        if (tid < FA_TILE) {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, n);
            }
            if (lane == 31) wmax[warp] = incl;
        }
        __syncthreads();
        if (tid < FA_TILE) {
            float before = carry_M;
            for (int w = 0; w < warp; w++) before = fmaxf(before, wmax[w]);
            float excl = __shfl_up_sync(0xffffffffu, incl, 1);
            if (lane == 0) excl = -INFINITY;
            before = fmaxf(before, excl);
            float ms = 1.0f, vs = 0.0f;
            if (tid < np && s != -INFINITY) {
                if (s > before) {
                    ms = libm_expf(__fsub_rn(before, s));
                    vs = 1.0f;
                } else {
                    vs = libm_expf(__fsub_rn(s, before));
                }
            } else {
                ms = -1.0f;   // marks a skipped position
            }
            ms_s[tid] = ms;
            vs_s[tid] = vs;
        }
        __syncthreads();
        if (tid == 0) {
            float m = carry_M;
            for (int w = 0; w < 4; w++) m = fmaxf(m, wmax[w]);
            carry_M = m;
        }
        if (is_val) {
            for (int i = 0; i < np; i++) {
                const float ms = ms_s[i];
                if (ms < 0.0f) continue;
                if (ms != 1.0f) x = r16(__fmul_rn(x, ms));
                x = r16(__fmaf_rn(__half2float(v_s[i * d.dv + tid]), vs_s[i], x));
            }
        } else if (is_s) {
            for (int i = 0; i < np; i++) {
                const float ms = ms_s[i];
                if (ms < 0.0f) continue;
                S = __fmaf_rn(S, ms, vs_s[i]);
            }
        }
        __syncthreads();
    }
    // sinks: only the chunk that starts at position 0 (flash_attn.rs:661-690), in f32
    float M = carry_M;
    if (a.sinks && ic0 == 0) {
        const float sh = a.sinks[h];
        float ms = 1.0f, vs = 1.0f;
        if (sh > M) {
            ms = libm_expf(__fsub_rn(M, sh));
            if (is_val) x = __fmul_rn(x, ms);
            M = sh;
        } else {
            vs = libm_expf(__fsub_rn(sh, M));
        }
        if (is_s) S = __fadd_rn(__fmul_rn(S, ms), vs);
    }
    if (is_val) part[2 + tid] = x;
    if (is_s) { part[0] = M; part[1] = S; }
}

// merge of the chunk partials in chunk order + normalisation (flash_attn.rs:779-832);
// with one chunk this is the plain one_chunk normalisation (S_inv = S == 0 ? 0 : 1/S).
__global__ void fa_merge_kernel(FaDims d, const float *__restrict__ partials, float *__restrict__ dst, bool split) {
    const int64_t row = blockIdx.x;
    const int e = threadIdx.x;
    if (e >= d.dv) return;
    const float *p0 = partials + row * d.n_chunks * (2 + d.dv);
    if (!split) {
        const float S = p0[1];
        const float s_inv = S == 0.0f ? 0.0f : __fdiv_rn(1.0f, S);
        dst[row * d.dv + e] = __fmul_rn(p0[2 + e], s_inv);
        return;
    }
    float fin = 0.0f, Mf = -INFINITY, Sf = 0.0f;
    for (int c = 0; c < d.n_chunks; c++) {
        if ((int64_t)c * d.chunk >= d.n_kv) continue;
        const float *p = p0 + (int64_t)c * (2 + d.dv);
        const float Mc = p[0], Sc = p[1];
        if (Sc == 0.0f) continue;
        const float Mn = fmaxf(Mf, Mc);
        const float so = libm_expf(__fsub_rn(Mf, Mn)), sn = libm_expf(__fsub_rn(Mc, Mn));
        fin = __fmaf_rn(fin, so, __fmul_rn(p[2 + e], sn));
        Sf = __fmaf_rn(Sf, so, __fmul_rn(Sc, sn));
        Mf = Mn;
    }
    if (Sf != 0.0f) fin = __fmul_rn(fin, __fdiv_rn(1.0f, Sf));
    dst[row * d.dv + e] = fin;
}


// ---------------------------------------------------------------------------
// One query row (a decode step): scores, chunk scan and merge in ONE kernel.
// Grid (chunk, head), block = 128 position / value threads + 1 warp for the S chain.  Per 128-position
// tile a thread first computes its position's score (the K row sits in its registers), then the tile runs
// exactly as in fa_rows_kernel.  The CTA that finishes a head's last chunk (a per-head counter tells)
// merges the chunk partials in chunk order and writes the row.  Same operations in the same order as the
// three-kernel path, so the same bits.
// ---------------------------------------------------------------------------
template <int DK>
__global__ void __launch_bounds__(160)
fa_decode_kernel(b200_flash_attn_args a, FaDims d, float kq_scale, float *__restrict__ partials, int *__restrict__ counters, bool split) {
    extern __shared__ __align__(16) unsigned char fsm[];
    __half *v_s = (__half *)fsm;                                  // [FA_TILE][dv]
    float *ms_s = (float *)(fsm + (size_t)FA_TILE * d.dv * 2);    // [FA_TILE]
    float *vs_s = ms_s + FA_TILE;
    float *wmax = vs_s + FA_TILE;                                 // [4] warp maxima
    float *q_s = wmax + 4;                                        // [DK], q rounded to f16
    double *tab_s = (double *)(q_s + DK);                         // [32] the exp2 table of libm_expf
    __shared__ float carry_M;
    __shared__ int is_last;
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c = blockIdx.x, h = blockIdx.y;
    const int hkv = h / (d.H / d.H_kv);
    const int64_t ic0 = (int64_t)c * d.chunk;
    const int64_t ic1 = ic0 + d.chunk < d.n_kv ? ic0 + d.chunk : d.n_kv;
    const int64_t row = h;
    float *part = partials + (row * d.n_chunks + c) * (2 + d.dv);
    const uint8_t *vbase = (const uint8_t *)a.v + (int64_t)hkv * a.v_nb2;
    const uint8_t *kbase = (const uint8_t *)a.k + (int64_t)hkv * a.k_nb2;
    float x = 0.0f, S = 0.0f;
    const bool is_val = tid < d.dv;
    const bool is_s = tid == 128;
    pdl_wait();   // q, and the cache rows the previous kernels wrote
    if (ic0 < d.n_kv) {
        const float *q = (const float *)((const uint8_t *)a.q + (int64_t)h * a.q_nb2);
        for (int i = tid; i < DK; i += blockDim.x) q_s[i] = r16(q[i]);
        if (tid >= 128) tab_s[tid - 128] = c_exp2_tab[tid - 128];
        if (tid == 0) carry_M = -INFINITY;
        // ALiBi slope of head h: crates/ggml/src/flash_attn.rs:356-370
        float slope = 1.0f;
        if (a.mask && a.max_bias > 0.0f) {
            const unsigned nl2 = 1u << (31 - __clz((unsigned)d.H));
            const float m0 = powf(2.0f, -a.max_bias / (float)nl2);
            const float m1 = powf(2.0f, -(a.max_bias / 2.0f) / (float)nl2);
            const float base = (unsigned)h < nl2 ? m0 : m1;
            const int ex = (unsigned)h < nl2 ? h + 1 : 2 * (h - (int)nl2) + 1;
            float acc = 1.0f, b = base;   // powi by repeated squaring
            for (int e2 = ex; e2 > 0; e2 >>= 1) {
                if (e2 & 1) acc = __fmul_rn(acc, b);
                b = __fmul_rn(b, b);
            }
            slope = acc;
        }
        __syncthreads();
        for (int64_t p0 = ic0; p0 < ic1; p0 += FA_TILE) {
            const int np = ic1 - p0 < FA_TILE ? (int)(ic1 - p0) : FA_TILE;
            // stage the V tile: np rows of dv halves, 16 bytes per load
            const int chunks_per_row = d.dv / 8;
            for (int i = tid; i < np * chunks_per_row; i += blockDim.x) {
                const int pr = i / chunks_per_row, cc = i % chunks_per_row;
                // asynchronous 16-byte copies: they land while the scores are computed
                const unsigned dst = (unsigned)__cvta_generic_to_shared(v_s + pr * d.dv + cc * 8);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(vbase + (p0 + pr) * a.v_nb1 + cc * 16) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            // this thread's position: the f16 dot of crates/ggml/src/vec_dot.rs:1982-2019, scale, softcap, mask
            float s = -INFINITY;
            if (tid < FA_TILE && tid < np) {
                const int64_t p = p0 + tid;
                __half2 kr[DK / 2];
                const uint4 *src = (const uint4 *)(kbase + p * a.k_nb1);
#pragma unroll
                for (int i = 0; i < DK / 8; i++) {
                    const uint4 v = src[i];
                    kr[4 * i + 0] = *(const __half2 *)&v.x;
                    kr[4 * i + 1] = *(const __half2 *)&v.y;
                    kr[4 * i + 2] = *(const __half2 *)&v.z;
                    kr[4 * i + 3] = *(const __half2 *)&v.w;
                }
                float val[16];
#pragma unroll
                for (int l = 0; l < 16; l++) {
                    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                    for (int cc = 0; cc < DK / 64; cc++) {
                        const int e = 64 * cc + l;
                        const float k0 = (e & 1) ? __high2float(kr[e >> 1]) : __low2float(kr[e >> 1]);
                        const float k1 = ((e + 16) & 1) ? __high2float(kr[(e + 16) >> 1]) : __low2float(kr[(e + 16) >> 1]);
                        const float k2 = ((e + 32) & 1) ? __high2float(kr[(e + 32) >> 1]) : __low2float(kr[(e + 32) >> 1]);
                        const float k3 = ((e + 48) & 1) ? __high2float(kr[(e + 48) >> 1]) : __low2float(kr[(e + 48) >> 1]);
                        s0 = __fmaf_rn(q_s[e], k0, s0);
                        s1 = __fmaf_rn(q_s[e + 16], k1, s1);
                        s2 = __fmaf_rn(q_s[e + 32], k2, s2);
                        s3 = __fmaf_rn(q_s[e + 48], k3, s3);
                    }
                    val[l] = __fadd_rn(__fadd_rn(s0, s2), __fadd_rn(s1, s3));
                }
#pragma unroll
                for (int half = 8; half >= 1; half >>= 1)
#pragma unroll
                    for (int i = 0; i < half; i++) val[i] = __fadd_rn(val[i], val[i + half]);
                s = __fmul_rn(val[0], kq_scale);
                if (a.logit_softcap != 0.0f) s = __fmul_rn(a.logit_softcap, tanhf(s));
                if (a.mask) {
                    const __half mh = ((const __half *)a.mask)[p];
                    const float mv = __fmul_rn(slope, __half2float(mh));
                    s = (mv == -INFINITY) ? -INFINITY : __fadd_rn(s, mv);
                }
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            // exclusive prefix maximum of the tile's scores (threads 0..127 = positions)
            float incl = s;
            if (tid < FA_TILE) {
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float n = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl = fmaxf(incl, n);
                }
                if (lane == 31) wmax[warp] = incl;
            }
            __syncthreads();
            if (tid < FA_TILE) {
                float before = carry_M;
                for (int w = 0; w < warp; w++) before = fmaxf(before, wmax[w]);
                float excl = __shfl_up_sync(0xffffffffu, incl, 1);
                if (lane == 0) excl = -INFINITY;
                before = fmaxf(before, excl);
                float ms = 1.0f, vs = 0.0f;
                if (tid < np && s != -INFINITY) {
                    if (s > before) {
                        ms = libm_expf_tab(__fsub_rn(before, s), tab_s);
                        vs = 1.0f;
                    } else {
                        vs = libm_expf_tab(__fsub_rn(s, before), tab_s);
                    }
                } else {
                    ms = -1.0f;   // marks a skipped position
                }
                ms_s[tid] = ms;
                vs_s[tid] = vs;
            }
            __syncthreads();
            if (tid == 0) {
                float m = carry_M;
                for (int w = 0; w < 4; w++) m = fmaxf(m, wmax[w]);
                carry_M = m;
            }
            if (is_val) {
#pragma unroll 4
                for (int i = 0; i < np; i++) {
                    const float ms = ms_s[i], vs = vs_s[i];
                    const float v = __half2float(v_s[i * d.dv + tid]);
                    if (ms == 1.0f) {            // no new maximum: one fma, one rounding
                        x = r16_fast(__fmaf_rn(v, vs, x));
                    } else if (ms >= 0.0f) {
                        x = r16(__fmul_rn(x, ms));
                        x = r16(__fmaf_rn(v, vs, x));
                    }                            // ms < 0: a skipped position
                }
            } else if (is_s) {
                for (int i = 0; i < np; i++) {
                    const float ms = ms_s[i];
                    if (ms < 0.0f) continue;
                    S = __fmaf_rn(S, ms, vs_s[i]);
                }
            }
            __syncthreads();
        }
        // sinks: only the chunk that starts at position 0 (flash_attn.rs:661-690), in f32
        float M = carry_M;
        if (a.sinks && ic0 == 0) {
            const float sh = a.sinks[h];
            float ms = 1.0f, vs = 1.0f;
            if (sh > M) {
                ms = libm_expf(__fsub_rn(M, sh));
                if (is_val) x = __fmul_rn(x, ms);
                M = sh;
            } else {
                vs = libm_expf(__fsub_rn(sh, M));
            }
            if (is_s) S = __fadd_rn(__fmul_rn(S, ms), vs);
        }
        if (is_val) part[2 + tid] = x;
        if (is_s) { part[0] = M; part[1] = S; }
    } else if (tid == 0) {   // out-of-range chunk: M = -inf, S = 0 (flash_attn.rs:757-764)
        part[0] = -INFINITY;
        part[1] = 0.0f;
    }
    // the CTA that completes the head merges its chunks
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(&counters[h], 1) == d.n_chunks - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (tid == 0) counters[h] = 0;   // ready for the next launch
    const int e = tid;
    const volatile float *p0 = partials + row * d.n_chunks * (2 + d.dv);
    if (!split) {
        if (e >= d.dv) return;
        const float Sv = p0[1];
        const float s_inv = Sv == 0.0f ? 0.0f : __fdiv_rn(1.0f, Sv);
        a.dst[row * d.dv + e] = __fmul_rn(p0[2 + e], s_inv);
        return;
    }
    // merge in chunk order (flash_attn.rs:744-859).  The exponentials depend only on the chunks' maxima: thread 0
    // walks those (the running maximum before and after each chunk), thread c takes chunk c's two exponentials,
    // and the value threads are left with the chain of fused multiply-adds.  so < 0 marks a chunk to skip.
    float *so_s = ms_s, *sn_s = vs_s;   // the tile arrays are free now
    const bool wide = d.n_chunks <= FA_TILE;
    if (wide) {
        if (tid == 0) {
            float Mf = -INFINITY;
            for (int cc = 0; cc < d.n_chunks; cc++) {
                const volatile float *p = p0 + (int64_t)cc * (2 + d.dv);
                const bool used = (int64_t)cc * d.chunk < d.n_kv && p[1] != 0.0f;
                const float Mc = p[0];
                const float Mn = used ? fmaxf(Mf, Mc) : Mf;
                so_s[cc] = used ? __fsub_rn(Mf, Mn) : 1.0f;   // arguments of the exponentials; a positive one marks "skip"
                sn_s[cc] = used ? __fsub_rn(Mc, Mn) : 1.0f;
                Mf = Mn;
            }
        }
        __syncthreads();
        float eo = -1.0f, en = -1.0f;
        if (tid < d.n_chunks && !(sn_s[tid] > 0.0f)) {
            eo = libm_expf(so_s[tid]);
            en = libm_expf(sn_s[tid]);
        }
        __syncthreads();
        if (tid < d.n_chunks) {
            so_s[tid] = eo;
            sn_s[tid] = en;
        }
        __syncthreads();
    }
    if (e >= d.dv) return;
    float fin = 0.0f, Mf = -INFINITY, Sf = 0.0f;
    for (int cc = 0; cc < d.n_chunks; cc++) {
        const volatile float *p = p0 + (int64_t)cc * (2 + d.dv);
        float so, sn;
        if (wide) {
            so = so_s[cc];
            sn = sn_s[cc];
            if (sn < 0.0f) continue;
        } else {
            if ((int64_t)cc * d.chunk >= d.n_kv) continue;
            const float Mc = p[0];
            if (p[1] == 0.0f) continue;
            const float Mn = fmaxf(Mf, Mc);
            so = libm_expf(__fsub_rn(Mf, Mn));
            sn = libm_expf(__fsub_rn(Mc, Mn));
            Mf = Mn;
        }
        fin = __fmaf_rn(fin, so, __fmul_rn(p[2 + e], sn));
        Sf = __fmaf_rn(Sf, so, __fmul_rn(p[1], sn));
    }
    if (Sf != 0.0f) fin = __fmul_rn(fin, __fdiv_rn(1.0f, Sf));
    a.dst[row * d.dv + e] = fin;
}

// per-device head counters of fa_decode_kernel (zero between launches)
static int *g_fa_counters[64] = {nullptr};
constexpr int FA_DECODE_MAX_HEADS = 4096;

static int flash_attn_decode_one_kernel(const b200_flash_attn_args *a, const FaDims &d, bool split, cudaStream_t s) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "flash_attn_ext: device index %d out of range", dev);
    if (!g_fa_counters[dev]) {
        B200_CUDA(cudaMalloc((void **)&g_fa_counters[dev], FA_DECODE_MAX_HEADS * sizeof(int)));
        B200_CUDA(cudaMemset(g_fa_counters[dev], 0, FA_DECODE_MAX_HEADS * sizeof(int)));
    }
    const size_t part_b = (size_t)d.H * d.n_chunks * (2 + d.dv) * 4;
    void *scratch = nullptr;
    int rc = scratch_get(part_b, &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const float kq_scale = a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
    const dim3 grid((unsigned)d.n_chunks, (unsigned)d.H);
    const size_t smem = (size_t)FA_TILE * d.dv * 2 + (2 * FA_TILE + 4 + d.dk) * 4 + 32 * 8;
    if (d.dk == 128)
        return launch_pdl(fa_decode_kernel<128>, grid, dim3(160), smem, s, *a, d, kq_scale, (float *)scratch, g_fa_counters[dev], split);
    return launch_pdl(fa_decode_kernel<64>, grid, dim3(160), smem, s, *a, d, kq_scale, (float *)scratch, g_fa_counters[dev], split);
}

static int check_args(const b200_flash_attn_args *a) {
    B200_REQUIRE(a != nullptr, "flash_attn_ext: null argument block");
    B200_REQUIRE(a->q && a->k && a->v && a->dst, "flash_attn_ext: null tensor pointer");
    B200_REQUIRE(a->n_tok >= 0 && a->n_kv >= 0 && a->n_head > 0 && a->n_head_kv > 0, "flash_attn_ext: bad shape");
    B200_REQUIRE(a->n_head % a->n_head_kv == 0, "flash_attn_ext: n_head %% n_head_kv != 0");
    B200_REQUIRE(a->dk == 64 || a->dk == 128, "flash_attn_ext: head size dk = %lld is not supported (64, 128)",
                 (long long)a->dk);
    B200_REQUIRE(a->dv == 64 || a->dv == 128, "flash_attn_ext: value size dv = %lld is not supported (64, 128)",
                 (long long)a->dv);
    B200_REQUIRE(a->k_nb1 % 16 == 0 && a->k_nb2 % 16 == 0 && a->v_nb1 % 16 == 0 && a->v_nb2 % 16 == 0 &&
                     ((uintptr_t)a->k & 15) == 0 && ((uintptr_t)a->v & 15) == 0,
                 "flash_attn_ext: k/v rows must be 16-byte aligned");
    B200_REQUIRE(!(a->max_bias > 0.0f) || a->mask, "flash_attn_ext: max_bias > 0 needs a mask");
    return B200_STATUS_SUCCESS;
}

int flash_attn_faithful_tiled(const b200_flash_attn_args *a, cudaStream_t s);   // flash_attn_tiled.cu
bool flash_attn_decode_head(const b200_flash_attn_args *a, int n_chunks, int64_t chunk, cudaStream_t s, int *rc);   // flash_attn_head.cu
bool flash_attn_rows_visible(const b200_flash_attn_args *a, cudaStream_t s, int *rc);                               // flash_attn_vis.cu
bool flash_attn_fast_rows(const b200_flash_attn_args *a, cudaStream_t s, int *rc);                                  // flash_attn_fast.cu
bool flash_attn_fast_prefill(const b200_flash_attn_args *a, cudaStream_t s, int *rc);                               // flash_attn_prefill.cu
bool flash_attn_fast_prefill_tc(const b200_flash_attn_args *a, cudaStream_t s, int *rc);                            // flash_attn_prefill_tc.cu
bool flash_attn_decode_mma(const b200_flash_attn_args *a, cudaStream_t s, int *rc);                                 // flash_attn_decode_mma.cu

// B200_FA_DECODE_MMA=0 keeps fast-mode attention of fewer than 64 query rows off the tensor-core flash-decoding kernel: single
// rows then take the CUDA-core kernel (the one the persistent decode step carries), several rows the exact kernels
// (read per call)
static bool fa_decode_mma_enabled() {
    const char *e = getenv("B200_FA_DECODE_MMA");
    return !(e && e[0] == '0');
}

// B200_FA_PREFILL_TC=1 sends fast-mode prompt attention with head size 128 to the tcgen05 kernel (read per call).  It gives
// the same values as the mma.sync kernel and, measured on 512 query rows over 32768 cached positions, the same speed
// (1.33 against 1.31 ms): with unswizzled core-matrix operands an M 128 x N 64 x K 16 MMA takes about 127 cycles and the
// 16-byte cp.async copies that build those operands cost their warps about 90 cycles each, so the mma.sync kernel stays
// the default until the operands come in through tensor-map copies in the 128-byte swizzle.
static bool fa_prefill_tc_enabled() {
    const char *e = getenv("B200_FA_PREFILL_TC");
    return e && e[0] == '1';
}

// B200_FA_DECODE_FUSED=0 keeps single-row attention on the three-kernel path (for side-by-side measurements)
static bool fa_decode_one_kernel_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_FA_DECODE_FUSED");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

int flash_attn_faithful_rows(const b200_flash_attn_args *a, cudaStream_t s) {
    FaDims d;
    d.dk = (int)a->dk; d.dv = (int)a->dv; d.T = (int)a->n_tok; d.H = (int)a->n_head; d.H_kv = (int)a->n_head_kv;
    d.n_kv = a->n_kv;
    const bool split = a->n_tok == 1 && a->n_kv >= 512;   // flash_attn.rs:931-939
    d.n_chunks = split ? (a->n_chunks > 0 ? a->n_chunks : 8) : 1;
    d.chunk = (a->n_kv + d.n_chunks - 1) / d.n_chunks;
    const int64_t rows = (int64_t)d.T * d.H;
    if (rows == 0) return B200_STATUS_SUCCESS;
    if (a->n_kv == 0) {
        B200_CUDA(cudaMemsetAsync(a->dst, 0, (size_t)rows * d.dv * 4, s));
        return B200_STATUS_SUCCESS;
    }
    B200_REQUIRE(d.T <= 65535 && d.H <= 65535, "flash_attn_ext: too many rows for one launch");
    if (d.T >= 2) {   // a few rows over a masked cache (batched decode): walk each row's visible positions only
        int rc = B200_STATUS_SUCCESS;
        if (flash_attn_rows_visible(a, s, &rc)) return rc;
    }
    if (d.T == 1 && split) {   // a chat-length context: one CTA per head, one warp per chunk
        int rc = B200_STATUS_SUCCESS;
        if (flash_attn_decode_head(a, d.n_chunks, d.chunk, s, &rc)) return rc;
    }
    if (d.T == 1 && d.H <= FA_DECODE_MAX_HEADS && fa_decode_one_kernel_enabled()) return flash_attn_decode_one_kernel(a, d, split, s);
    const size_t score_b = ((size_t)rows * d.n_kv * 4 + 255) / 256 * 256;
    const size_t part_b = (size_t)rows * d.n_chunks * (2 + d.dv) * 4;
    void *scratch = nullptr;
    int rc = scratch_get(score_b + part_b, &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    float *scores = (float *)scratch;
    float *partials = (float *)((uint8_t *)scratch + score_b);
    const float kq_scale = a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
    dim3 g1((unsigned)((d.n_kv + 127) / 128), (unsigned)d.H_kv);
    const size_t sm1 = (size_t)8 * d.dk * 4;
    if (d.dk == 128) fa_scores_kernel<128><<<g1, 128, sm1, s>>>(*a, d, kq_scale, scores);
    else fa_scores_kernel<64><<<g1, 128, sm1, s>>>(*a, d, kq_scale, scores);
    B200_CUDA(cudaGetLastError());
    dim3 g2((unsigned)d.n_chunks, (unsigned)d.H, (unsigned)d.T);
    const size_t sm2 = (size_t)FA_TILE * d.dv * 2 + (2 * FA_TILE + 4) * 4;
    fa_rows_kernel<<<g2, 160, sm2, s>>>(*a, d, scores, partials);
    B200_CUDA(cudaGetLastError());
    fa_merge_kernel<<<(unsigned)rows, 128, 0, s>>>(d, partials, a->dst, split);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

}  // namespace b200

extern "C" int b200_flash_attn_ext(const struct b200_flash_attn_args *args, void *stream) {
    using namespace b200;
    int rc = check_args(args);
    if (rc != B200_STATUS_SUCCESS) return rc;
    // mode 1 asks for the fast kernels wherever they apply; so does the fast numerics policy (mode 0) for the tensor-core
    // decode kernel.  The CUDA-core kernel takes single query rows only under the policy: for several rows over a shared
    // cache, each seeing a small part of it, the exact kernels that walk per-row lists of visible positions are quicker
    // than it (measured on 16 sequences over 10240 cells).
    const bool policy = args->mode == 0 && numerics_mode() == 1;
    if ((args->mode == 1 || policy) && args->n_tok < 64) {
        if (fa_decode_mma_enabled() && flash_attn_decode_mma(args, (cudaStream_t)stream, &rc)) return rc;
        if ((args->mode == 1 || args->n_tok == 1) && flash_attn_fast_rows(args, (cudaStream_t)stream, &rc)) return rc;
    }
    if (args->n_tok < 64) return flash_attn_faithful_rows(args, (cudaStream_t)stream);
    // prompt batches: the tensor-core kernel under mode 1 or the fast numerics policy, the bit-exact tiled kernel otherwise
    if (args->mode == 1 || (args->mode == 0 && numerics_mode() == 1)) {
        if (fa_prefill_tc_enabled() && flash_attn_fast_prefill_tc(args, (cudaStream_t)stream, &rc)) return rc;   // head size 128, tcgen05
        if (flash_attn_fast_prefill(args, (cudaStream_t)stream, &rc)) return rc;
    }
    return flash_attn_faithful_tiled(args, (cudaStream_t)stream);
}
