// FLASH_ATTN_EXT for a few query rows over a cache most of which each row does not see (batched decode over
// the unified KV cache: 16 sequences share the cells, a token's mask hides the other fifteen's).
//
// The CPU skips a masked position before it does anything with it (crates/ggml/src/flash_attn.rs:482-560), so a
// row's result is the online softmax over its visible positions in ascending order and nothing else.  The
// three-kernel path of flash_attn.cu still walks every position of every row to find that out.  Here a first
// kernel writes each row's visible positions as a list (ordered compaction of the mask row), the score kernel
// computes dots for list entries only, and the scan kernel walks the list: the same operations on the same
// values in the same order, a sixteenth of the work when sixteen sequences share the cache.
#include <cmath>
#include <cstdlib>

#include "common.cuh"
#include "fa_math.cuh"

namespace b200 {

namespace {

constexpr int FV_TILE = 128;

__device__ __forceinline__ float v_r16(float v) { return __half2float(__float2half_rn(v)); }
// the same rounding for the long dependent chain: inside the normal f16 range, round to nearest even at bit 13 of
// the f32 pattern with three integer operations; everything else takes the conversion pair
__device__ __forceinline__ float v_r16_fast(float v) {
    const uint32_t b = __float_as_uint(v);
    if (((b & 0x7fffffffu) - 0x38800000u) < (0x477ff000u - 0x38800000u))
        return __uint_as_float((b + 0x0fffu + ((b >> 13) & 1u)) & 0xffffe000u);
    return v_r16(v);
}

// vis[t][0 .. nvis[t]) = the positions of mask row t that are not -inf, ascending
__global__ void __launch_bounds__(256)
fa_visible_kernel(const uint8_t *__restrict__ mask, int64_t mask_nb1, int64_t n_kv, int32_t *__restrict__ vis, int32_t *__restrict__ nvis) {
    __shared__ int wsum[8];
    __shared__ int base_s;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint16_t *row = (const uint16_t *)(mask + (int64_t)t * mask_nb1);
    int32_t *out = vis + (int64_t)t * n_kv;
    if (tid == 0) base_s = 0;
    __syncthreads();
    for (int64_t p0 = 0; p0 < n_kv; p0 += 256) {
        const int64_t p = p0 + tid;
        const bool seen = p < n_kv && row[p] != 0xFC00u;   // f16 -inf
        const unsigned bal = __ballot_sync(0xffffffffu, seen);
        if (lane == 0) wsum[warp] = __popc(bal);
        __syncthreads();
        int before = base_s;
        for (int w = 0; w < warp; w++) before += wsum[w];
        if (seen) out[before + __popc(bal & ((1u << lane) - 1u))] = (int32_t)p;
        __syncthreads();
        if (tid == 0) {
            int s = base_s;
            for (int w = 0; w < 8; w++) s += wsum[w];
            base_s = s;
        }
        __syncthreads();
    }
    if (tid == 0) nvis[t] = base_s;
}

// scores[(t * H + h) * n_kv + i] for list entry i of row t: the f16 dot of crates/ggml/src/vec_dot.rs:1982-2019
// with q rounded to f16, scale, softcap, slope * mask.  grid (list tiles, kv heads, rows): the K row of an entry
// serves the H / H_kv heads of its group.
template <int DK>
__global__ void __launch_bounds__(128)
fa_scores_vis_kernel(b200_flash_attn_args a, int H, int H_kv, int64_t n_kv, float kq_scale, const int32_t *__restrict__ vis,
                     const int32_t *__restrict__ nvis, float *__restrict__ scores) {
    extern __shared__ float q_s[];   // [group][DK], q rounded to f16
    pdl_trigger();
    pdl_wait();
    const int group = H / H_kv;
    const int hkv = blockIdx.y, t = blockIdx.z;
    const int n = nvis[t];
    if ((int64_t)blockIdx.x * 128 >= n) return;
    for (int i = threadIdx.x; i < group * DK; i += 128) {
        const int h = hkv * group + i / DK;
        const float *q = (const float *)((const uint8_t *)a.q + (int64_t)t * a.q_nb1 + (int64_t)h * a.q_nb2);
        q_s[i] = v_r16(q[i % DK]);
    }
    __syncthreads();
    const int64_t i = (int64_t)blockIdx.x * 128 + threadIdx.x;
    if (i >= n) return;
    const int64_t p = vis[(int64_t)t * n_kv + i];
    __half2 kr[DK / 2];
    const uint4 *src = (const uint4 *)((const uint8_t *)a.k + p * a.k_nb1 + (int64_t)hkv * a.k_nb2);
#pragma unroll
    for (int j = 0; j < DK / 8; j++) {
        const uint4 v = src[j];
        kr[4 * j + 0] = *(const __half2 *)&v.x;
        kr[4 * j + 1] = *(const __half2 *)&v.y;
        kr[4 * j + 2] = *(const __half2 *)&v.z;
        kr[4 * j + 3] = *(const __half2 *)&v.w;
    }
    const float mval = __half2float(((const __half *)((const uint8_t *)a.mask + (int64_t)t * a.mask_nb1))[p]);
    for (int g = 0; g < group; g++) {
        const int h = hkv * group + g;
        const float *q = q_s + g * DK;
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
            for (int j = 0; j < half; j++) val[j] = __fadd_rn(val[j], val[j + half]);
        float s = __fmul_rn(val[0], kq_scale);
        if (a.logit_softcap != 0.0f) s = __fmul_rn(a.logit_softcap, tanhf(s));
        float slope = 1.0f;
        if (a.max_bias > 0.0f) {
            // ALiBi slope of head h: crates/ggml/src/flash_attn.rs:356-370
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
        const float mv = __fmul_rn(slope, mval);
        s = (mv == -INFINITY) ? -INFINITY : __fadd_rn(s, mv);
        scores[((int64_t)t * H + h) * n_kv + i] = s;
    }
}

// One CTA per (head, row): the online softmax over the row's list, tile by tile (prefix maxima, one exponential
// per entry, then the sequential f16 accumulation with one thread per value element), normalised at the end
// (one chunk: out = VKQ * (S == 0 ? 0 : 1 / S), flash_attn.rs:694-720).
__global__ void __launch_bounds__(160)
fa_rows_vis_kernel(b200_flash_attn_args a, int H, int H_kv, int dv, int64_t n_kv, const int32_t *__restrict__ vis,
                   const int32_t *__restrict__ nvis, const float *__restrict__ scores) {
    extern __shared__ __align__(16) unsigned char fsm[];
    __half *v_s = (__half *)fsm;                                  // [FV_TILE][dv]
    float *ms_s = (float *)(fsm + (size_t)FV_TILE * dv * 2);      // [FV_TILE]
    float *vs_s = ms_s + FV_TILE;
    float *wmax = vs_s + FV_TILE;                                 // [4] warp maxima
    __shared__ float carry_M, S_fin;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.x, t = blockIdx.y;
    const int hkv = h / (H / H_kv);
    const int64_t row = (int64_t)t * H + h;
    const int n = nvis[t];
    const float *srow = scores + row * n_kv;
    const int32_t *list = vis + (int64_t)t * n_kv;
    const uint8_t *vbase = (const uint8_t *)a.v + (int64_t)hkv * a.v_nb2;
    if (tid == 0) carry_M = -INFINITY;
    float x = 0.0f, S = 0.0f;
    const bool is_val = tid < dv;
    const bool is_s = tid == 128;
    __syncthreads();
    for (int p0 = 0; p0 < n; p0 += FV_TILE) {
        const int np = n - p0 < FV_TILE ? n - p0 : FV_TILE;
        float s = -INFINITY;
        if (tid < np) s = srow[p0 + tid];
        const int chunks_per_row = dv / 8;
        for (int i = tid; i < np * chunks_per_row; i += blockDim.x) {
            const int pr = i / chunks_per_row, cc = i % chunks_per_row;
            const uint4 v = *(const uint4 *)(vbase + (int64_t)list[p0 + pr] * a.v_nb1 + cc * 16);
            *(uint4 *)(v_s + pr * dv + cc * 8) = v;
        }
        float incl = s;
        if (tid < FV_TILE) {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float nb = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl = fmaxf(incl, nb);
            }
            if (lane == 31) wmax[warp] = incl;
        }
        __syncthreads();
        if (tid < FV_TILE) {
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
                ms = -1.0f;   // marks a skipped entry
            }
            ms_s[tid] = ms;
            vs_s[tid] = vs;
        }
        __syncthreads();
        if (tid == 0) {
            float mx = carry_M;
            for (int w = 0; w < 4; w++) mx = fmaxf(mx, wmax[w]);
            carry_M = mx;
        }
        if (is_val) {
            for (int i = 0; i < np; i++) {
                const float ms = ms_s[i];
                if (ms < 0.0f) continue;
                if (ms != 1.0f) x = v_r16(__fmul_rn(x, ms));
                x = v_r16_fast(__fmaf_rn(__half2float(v_s[i * dv + tid]), vs_s[i], x));
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
    // sinks (flash_attn.rs:661-690), in f32
    float M = carry_M;
    if (a.sinks) {
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
    if (is_s) S_fin = S;
    __syncthreads();
    if (is_val) {
        const float Sv = S_fin;
        const float s_inv = Sv == 0.0f ? 0.0f : __fdiv_rn(1.0f, Sv);
        a.dst[row * dv + tid] = __fmul_rn(x, s_inv);
    }
}

// B200_FA_VISIBLE=0 keeps few-row attention over a masked cache on the path that walks every position
bool fa_visible_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_FA_VISIBLE");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

}  // namespace

// Inside one graph_compute every layer's attention reads the same mask: the lists made for the first layer serve
// the others.  The backend brackets a node list with flash_attn_graph_scope(true / false); outside such a scope
// (the op-level entry point, where a caller may rewrite a mask in place between calls) nothing is reused.
static thread_local unsigned long long t_scope = 0;
static unsigned long long g_scope_counter = 0;
struct VisibleCache {
    unsigned long long scope = 0;
    const void *mask = nullptr;
    int64_t nb1 = 0, n_kv = 0, T = 0;
    int32_t *vis = nullptr, *nvis = nullptr;
};
static VisibleCache g_vis_cache[64];
void flash_attn_graph_scope(bool enter) { t_scope = enter ? ++g_scope_counter : 0; }

// true when the launches were made; false = not this path's case (the caller takes the other one)
bool flash_attn_rows_visible(const b200_flash_attn_args *a, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (!fa_visible_enabled() || !a->mask || a->n_tok < 2 || a->n_kv < 1024 || a->n_kv > 0x7fffffffLL) return false;
    if (!((a->dk == 128 || a->dk == 64) && (a->dv == 128 || a->dv == 64))) return false;
    const int64_t T = a->n_tok, H = a->n_head, n_kv = a->n_kv;
    if (T > 65535 || H > 65535) return false;
    const size_t vis_b = ((size_t)T * n_kv * 4 + 255) / 256 * 256, nvis_b = ((size_t)T * 4 + 255) / 256 * 256;
    const size_t score_b = (size_t)T * H * n_kv * 4;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    void *scratch = nullptr, *lists = nullptr;
    *rc = scratch_get(score_b, &scratch);
    if (*rc == B200_STATUS_SUCCESS) *rc = scratch_get_lists(vis_b + nvis_b, &lists);   // its own block: the lists outlive this call
    if (*rc != B200_STATUS_SUCCESS) return true;
    int32_t *vis = (int32_t *)lists;
    int32_t *nvis = (int32_t *)((uint8_t *)lists + vis_b);
    float *scores = (float *)scratch;
    const float kq_scale = a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
    VisibleCache &vc = g_vis_cache[dev];
    const bool reuse = t_scope != 0 && vc.scope == t_scope && vc.mask == a->mask && vc.nb1 == a->mask_nb1 && vc.n_kv == n_kv && vc.T == T &&
                       vc.vis == vis && vc.nvis == nvis;
    if (!reuse) {
        *rc = launch_pdl(fa_visible_kernel, dim3((unsigned)T), dim3(256), 0, s, (const uint8_t *)a->mask, a->mask_nb1, n_kv, vis, nvis);
        if (*rc != B200_STATUS_SUCCESS) return true;
        vc.scope = t_scope; vc.mask = a->mask; vc.nb1 = a->mask_nb1; vc.n_kv = n_kv; vc.T = T; vc.vis = vis; vc.nvis = nvis;
    }
    const int group = (int)(H / a->n_head_kv);
    const dim3 g1((unsigned)((n_kv + 127) / 128), (unsigned)a->n_head_kv, (unsigned)T);
    const size_t sm1 = (size_t)group * a->dk * 4;
    if (a->dk == 128)
        *rc = launch_pdl(fa_scores_vis_kernel<128>, g1, dim3(128), sm1, s, *a, (int)H, (int)a->n_head_kv, n_kv, kq_scale, (const int32_t *)vis,
                         (const int32_t *)nvis, scores);
    else
        *rc = launch_pdl(fa_scores_vis_kernel<64>, g1, dim3(128), sm1, s, *a, (int)H, (int)a->n_head_kv, n_kv, kq_scale, (const int32_t *)vis,
                         (const int32_t *)nvis, scores);
    if (*rc != B200_STATUS_SUCCESS) return true;
    const size_t sm2 = (size_t)FV_TILE * a->dv * 2 + (2 * FV_TILE + 4) * 4;
    *rc = launch_pdl(fa_rows_vis_kernel, dim3((unsigned)H, (unsigned)T), dim3(160), sm2, s, *a, (int)H, (int)a->n_head_kv, (int)a->dv, n_kv,
                     (const int32_t *)vis, (const int32_t *)nvis, (const float *)scores);
    return true;
}

}  // namespace b200
