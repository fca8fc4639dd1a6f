// Single-row split-KV FLASH_ATTN_EXT with one CTA per head: every chunk of the CPU's chunked scan
// (crates/ggml/src/flash_attn.rs:744-859) is one warp, and the merge happens in shared memory.
//
// fa_decode_kernel (flash_attn.cu) gives each (chunk, head) its own CTA and lets the last CTA of a head
// merge the chunks through global memory.  At the context lengths of a chat (hundreds to a few thousand
// positions, 8 to 24 chunks) a chunk is a few dozen positions: a 160-thread CTA per chunk is mostly idle, and
// the partials' round trip through global memory (fence, atomic counter, re-read) and the merge, where every
// value thread recomputes the chunks' exponentials one after the other, are a large part of the kernel's
// latency.  Here a warp scans a chunk 32 positions at a time: lane l computes position l's score (the same f16
// dot, fold and tree), a shuffle scan gives the running maxima, each lane takes the one exponential of its
// position, and the lanes then walk the 32 positions together, each owning DV / 32 value elements.  The
// chunks' (M, S, VKQ) go to shared memory; chunk c's two merge exponentials are computed by thread c, and the
// value threads are left with the fused multiply-adds in chunk order.  Operation for operation the
// arithmetic is fa_decode_kernel's, so the output bits are the same.
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "fa_math.cuh"

namespace b200 {

namespace {

constexpr int FH_TILE = 32;          // positions per warp pass
constexpr int FH_MAX_CHUNKS = 16;    // warps per CTA: 512 threads leave each lane the registers of a 128-element K row

__device__ __forceinline__ float h_r16(float v) { return __half2float(__float2half_rn(v)); }
// round to nearest even at bit 13 of the f32 pattern inside the normal f16 range, the conversion pair elsewhere
__device__ __forceinline__ float h_r16_fast(float v) {
    const uint32_t b = __float_as_uint(v);
    if (((b & 0x7fffffffu) - 0x38800000u) < (0x477ff000u - 0x38800000u))
        return __uint_as_float((b + 0x0fffu + ((b >> 13) & 1u)) & 0xffffe000u);
    return h_r16(v);
}

}  // namespace

template <int DK, int DV>
__global__ void __launch_bounds__(FH_MAX_CHUNKS * 32)
fa_decode_head_kernel(b200_flash_attn_args a, int H, int H_kv, int64_t n_kv, int n_chunks, int64_t chunk, float kq_scale) {
    constexpr int E = DV / 32;                                        // value elements per lane
    extern __shared__ __align__(16) unsigned char hsm[];
    __half *v_all = (__half *)hsm;                                    // [n_chunks][FH_TILE][DV]
    float *part = (float *)(hsm + (size_t)n_chunks * FH_TILE * DV * 2);   // [n_chunks][2 + DV]
    float *so_s = part + (size_t)n_chunks * (2 + DV);                 // [n_chunks] merge scale of the running sums
    float *sn_s = so_s + n_chunks;                                    // [n_chunks] merge scale of the chunk
    float *q_s = sn_s + n_chunks;                                     // [DK] q rounded to f16
    double *tab_s = (double *)(q_s + DK);                             // [32] the exp2 table of libm_expf
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, c = tid >> 5;
    const int h = blockIdx.x;
    const int hkv = h / (H / H_kv);
    const uint8_t *vbase = (const uint8_t *)a.v + (int64_t)hkv * a.v_nb2;
    const uint8_t *kbase = (const uint8_t *)a.k + (int64_t)hkv * a.k_nb2;
    pdl_wait();   // q, and the cache rows the previous kernels wrote
    {
        const float *q = (const float *)((const uint8_t *)a.q + (int64_t)h * a.q_nb2);
        for (int i = tid; i < DK; i += blockDim.x) q_s[i] = h_r16(q[i]);
        if (tid < 32) tab_s[tid] = c_exp2_tab[tid];
    }
    // ALiBi slope of head h: crates/ggml/src/flash_attn.rs:356-370
    float slope = 1.0f;
    if (a.mask && a.max_bias > 0.0f) {
        const unsigned nl2 = 1u << (31 - __clz((unsigned)H));
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

    const int64_t ic0 = (int64_t)c * chunk;
    const int64_t ic1 = ic0 + chunk < n_kv ? ic0 + chunk : n_kv;
    float x[E], S = 0.0f, M = -INFINITY;
#pragma unroll
    for (int e = 0; e < E; e++) x[e] = 0.0f;
    __half *v_s = v_all + (size_t)c * FH_TILE * DV;
    for (int64_t p0 = ic0; p0 < ic1; p0 += FH_TILE) {
        const int np = ic1 - p0 < FH_TILE ? (int)(ic1 - p0) : FH_TILE;
        // stage the V rows of these positions: 16-byte asynchronous copies that land while the scores are computed
        for (int i = lane; i < np * (DV / 8); i += 32) {
            const int pr = i / (DV / 8), cc = i % (DV / 8);
            const unsigned dst = (unsigned)__cvta_generic_to_shared(v_s + pr * DV + cc * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(vbase + (p0 + pr) * a.v_nb1 + cc * 16) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        // lane = position: the f16 dot of crates/ggml/src/vec_dot.rs:1982-2019, scale, softcap, mask
        float s = -INFINITY;
        if (lane < np) {
            const int64_t p = p0 + lane;
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
        // running maximum before each position: the chunk's maximum so far, then the earlier lanes
        float incl = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float nb = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl = fmaxf(incl, nb);
        }
        float excl = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) excl = -INFINITY;
        const float before = fmaxf(M, excl);
        float ms = -1.0f, vs = 0.0f;   // ms < 0 marks a skipped position
        if (lane < np && s != -INFINITY) {
            if (s > before) {
                ms = libm_expf_tab(__fsub_rn(before, s), tab_s);
                vs = 1.0f;
            } else {
                ms = 1.0f;
                vs = libm_expf_tab(__fsub_rn(s, before), tab_s);
            }
        }
        M = fmaxf(M, __shfl_sync(0xffffffffu, incl, 31));
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncwarp();
        for (int i = 0; i < np; i++) {
            const float msi = __shfl_sync(0xffffffffu, ms, i), vsi = __shfl_sync(0xffffffffu, vs, i);
            if (msi < 0.0f) continue;
            float v[E];
            if constexpr (E == 4) {
                const uint2 raw = *(const uint2 *)(v_s + i * DV + 4 * lane);
                const __half2 lo = *(const __half2 *)&raw.x, hi = *(const __half2 *)&raw.y;
                v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
            } else {
                const __half2 lo = *(const __half2 *)(v_s + i * DV + 2 * lane);
                v[0] = __low2float(lo); v[1] = __high2float(lo);
            }
            if (msi == 1.0f) {               // no new maximum: one fma, one rounding
#pragma unroll
                for (int e = 0; e < E; e++) x[e] = h_r16_fast(__fmaf_rn(v[e], vsi, x[e]));
            } else {
#pragma unroll
                for (int e = 0; e < E; e++) {
                    x[e] = h_r16(__fmul_rn(x[e], msi));
                    x[e] = h_r16(__fmaf_rn(v[e], vsi, x[e]));
                }
            }
            S = __fmaf_rn(S, msi, vsi);
        }
        __syncwarp();   // the staged rows are overwritten by the next pass
    }
    // sinks: only the chunk that starts at position 0 (flash_attn.rs:661-690), in f32
    if (a.sinks && ic0 == 0 && ic0 < n_kv) {
        const float sh = a.sinks[h];
        float ms = 1.0f, vs = 1.0f;
        if (sh > M) {
            ms = libm_expf(__fsub_rn(M, sh));
#pragma unroll
            for (int e = 0; e < E; e++) x[e] = __fmul_rn(x[e], ms);
            M = sh;
        } else {
            vs = libm_expf(__fsub_rn(sh, M));
        }
        S = __fadd_rn(__fmul_rn(S, ms), vs);
    }
    {
        float *pc = part + (size_t)c * (2 + DV);
        if (lane == 0) {
            pc[0] = ic0 < n_kv ? M : -INFINITY;   // out-of-range chunk: M = -inf, S = 0 (flash_attn.rs:757-764)
            pc[1] = ic0 < n_kv ? S : 0.0f;
        }
#pragma unroll
        for (int e = 0; e < E; e++) pc[2 + E * lane + e] = x[e];
    }
    __syncthreads();
    // merge in chunk order: thread 0 walks the maxima (a few dozen comparisons) and leaves, for every chunk, the
    // maximum before and after it; thread c then takes chunk c's two exponentials; the value threads chain the fmas
    if (tid == 0) {
        float Mf = -INFINITY;
        for (int cc = 0; cc < n_chunks; cc++) {
            const float *p = part + (size_t)cc * (2 + DV);
            const bool used = (int64_t)cc * chunk < n_kv && p[1] != 0.0f;
            const float Mn = used ? fmaxf(Mf, p[0]) : Mf;
            so_s[cc] = used ? __fsub_rn(Mf, Mn) : 1.0f;    // arguments of the exponentials; a positive one marks "skip"
            sn_s[cc] = used ? __fsub_rn(p[0], Mn) : 1.0f;
            Mf = Mn;
        }
    }
    __syncthreads();
    if (tid < n_chunks) {
        const float ao = so_s[tid], an = sn_s[tid];
        const bool used = !(an > 0.0f);
        so_s[tid] = used ? libm_expf(ao) : -1.0f;
        sn_s[tid] = used ? libm_expf(an) : -1.0f;
    }
    __syncthreads();
    if (tid < DV) {
        float fin = 0.0f, Sf = 0.0f;
        for (int cc = 0; cc < n_chunks; cc++) {
            const float so = so_s[cc], sn = sn_s[cc];
            if (sn < 0.0f) continue;
            const float *p = part + (size_t)cc * (2 + DV);
            fin = __fmaf_rn(fin, so, __fmul_rn(p[2 + tid], sn));
            Sf = __fmaf_rn(Sf, so, __fmul_rn(p[1], sn));
        }
        if (Sf != 0.0f) fin = __fmul_rn(fin, __fdiv_rn(1.0f, Sf));
        a.dst[(int64_t)h * DV + tid] = fin;
    }
}

// B200_FA_DECODE_HEAD=1 sends single-row split-KV attention here.  Measured inside the 8B-shaped decode step it
// loses to the CTA-per-chunk kernel (2.79 against 2.40 ms per token at 768 cached positions): with one CTA per
// head only 32 SMs work, and each lane's K row is 32 uncoalesced 16-byte loads that one SM's load pipe now
// serves for all sixteen chunks.  It stays selectable until the K rows are staged through shared memory.
static bool fa_decode_head_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_FA_DECODE_HEAD");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// true when the launch was made; false = not this kernel's case (the caller takes the other path)
bool flash_attn_decode_head(const b200_flash_attn_args *a, int n_chunks, int64_t chunk, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (!fa_decode_head_enabled() || n_chunks < 2 || n_chunks > FH_MAX_CHUNKS || chunk > 2048) return false;
    if (!((a->dk == 128 && a->dv == 128) || (a->dk == 64 && a->dv == 64))) return false;
    const int dv = (int)a->dv, dk = (int)a->dk;
    const size_t smem = (size_t)n_chunks * FH_TILE * dv * 2 + ((size_t)n_chunks * (2 + dv) + 2 * n_chunks + dk) * 4 + 8 + 32 * 8;
    const float kq_scale = a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
    static bool attr_done[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!attr_done[dev]) {
        if (cudaFuncSetAttribute(fa_decode_head_kernel<128, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(fa_decode_head_kernel<64, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        attr_done[dev] = true;
    }
    if (smem > 220 * 1024) return false;
    const dim3 grid((unsigned)a->n_head), block((unsigned)n_chunks * 32);
    if (dk == 128)
        *rc = launch_pdl(fa_decode_head_kernel<128, 128>, grid, block, smem, s, *a, (int)a->n_head, (int)a->n_head_kv, a->n_kv, n_chunks, chunk, kq_scale);
    else
        *rc = launch_pdl(fa_decode_head_kernel<64, 64>, grid, block, smem, s, *a, (int)a->n_head, (int)a->n_head_kv, a->n_kv, n_chunks, chunk, kq_scale);
    return true;
}

}  // namespace b200
