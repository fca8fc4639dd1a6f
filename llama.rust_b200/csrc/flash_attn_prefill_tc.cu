// FLASH_ATTN_EXT, fast mode, prompt batches, head size 128: attention on the tcgen05 tensor cores.
//
// The same function and the same tolerance as flash_attn_prefill.cu (the mma.sync form, which stays for head size 64
// and for one query head per KV head):   softmax(q k^T * scale + mask) v   (crates/ggml/src/flash_attn.rs:482-736).
//   * a CTA takes 128 rows of one KV head, a row being (token, query head of the KV head's group) with the heads of a
//     token adjacent; row r is lane r of tensor memory, and two threads (warps w and w + 4 of the CTA's eight) own it, one
//     half of the columns each: the only thing a row's softmax exchanges is the two halves' maxima, through shared memory;
//   * per tile of 64 cached positions:  S = Q K^T  as eight tcgen05.mma.kind::f16 (M 128, N 64, K 16) from shared memory
//     into 64 tensor-memory columns; the threads read their rows with tcgen05.ld, apply scale and mask, keep the running
//     maximum and sum (exp2), round the weights to f16 into shared memory in the A-operand layout; then  P V  as four
//     MMAs (M 128, N 128, K 16) into 128 further columns, read back and folded into the f32 output half row each thread keeps
//     in registers (o = o * alpha + p v): nothing is ever rescaled inside tensor memory;
//   * operands are 8-row x 16-byte core matrices without swizzle.  Q and P are K-major A operands; K is a K-major B
//     operand (its rows are positions); V is an MN-major B operand: a cached row's 16-byte pieces (8 value elements of
//     one position) are exactly the rows of MN-major core matrices, so K and V tiles go to shared memory with the same
//     16-byte cp.async pattern and no transposition.  In a descriptor the leading-dimension offset is the distance
//     between core matrices that follow one another along K's 16-byte rows for a K-major operand, and between groups of
//     8 K-rows for an MN-major one (the stride-dimension offset is the other direction in both cases);
//   * the CTA is specialized by warp: eight compute warps (above); one warp whose first lane issues every MMA; two
//     warps that bring K tiles and their mask rows into shared memory (and decide, from the mask rows, whether anybody
//     sees the tile at all); one that brings V tiles.  They meet only at mbarriers: copies landed (k_full, v_full), MMAs
//     completed (s_done, o_done, and the buffers they free: k_free, v_free, p_free, via tcgen05.commit), rows read or
//     written by all 256 compute threads (s_free, p_full, pv_free).  Three buffers of K (with its mask rows), V, P and
//     of the score region, two of the p v region: the score MMAs run two tiles ahead of the softmax, and a tile's p v
//     has the next two softmaxes to complete before its result is folded into the output rows.  Every barrier advances once per tile whether or not the
//     tile is visible, so a buffer's phase is a function of the tile index alone;
//   * a tile none of the CTA's rows sees (the causal future) costs its K copy: no MMAs, no V copy, no softmax.
// Every mbarrier wait is bounded; a wait that runs out records code 4, and the CTA frees its tensor memory and leaves.
#include <cstdlib>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int TC_BM = 128, TC_BN = 64, TC_D = 128;
constexpr int TC_COMPUTE_WARPS = 8;   // two warps per quarter of the rows: each takes half of a row's columns
constexpr int TC_MMA_WARP = 8, TC_KLOAD_WARP = 9, TC_VLOAD_WARP = 10, TC_KLOAD_WARP2 = 11;   // two warps share the K tiles and mask rows
constexpr int TC_THREADS = 12 * 32;   // three warp groups: registers move between them with setmaxnreg
constexpr int TC_REGS_COMPUTE = 208, TC_REGS_CONTROL = 88;   // 2 x 128 x 208 + 128 x 88 = 64512 of the SM's 65536
constexpr int TC_MAX_TOK = TC_BM / 2 + 1;          // mask rows a CTA can span (two or more heads per KV head)
constexpr int TC_MPITCH = TC_BN * 2 + 16;
constexpr int TC_Q_BYTES = TC_BM * TC_D * 2;       // 32768
constexpr int TC_K_BYTES = TC_BN * TC_D * 2;       // 16384
constexpr int TC_P_BYTES = TC_BM * TC_BN * 2;      // 16384
constexpr int TC_M_BYTES = TC_MAX_TOK * TC_MPITCH; // 9360
constexpr int TC_NS = 3;                            // buffers of K (with its mask rows), V, P and of the score region: tile j uses j % 3
constexpr int TC_SMEM = TC_Q_BYTES + 2 * TC_NS * TC_K_BYTES + TC_NS * TC_P_BYTES + TC_NS * TC_M_BYTES + 1024;   // Q | K x 3 | V x 3 | P x 3 | mask x 3
constexpr int TC_TMEM_PV = 256;                     // tensor-memory columns: scores at 0, 64, 128; p v at 256 and 384 (tile j uses j % 2)
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;
constexpr float TC_LOG2E = 1.4426950408889634f;
// kind::f16 instruction descriptors: f32 accumulator, f16 x f16, M = 128; scores: N = 64, both operands K-major;
// p v: N = 128, B (the V tile) MN-major
constexpr uint32_t TC_IDESC_S = (1u << 4) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
constexpr uint32_t TC_IDESC_O = (1u << 4) | (1u << 16) | ((uint32_t)(TC_D >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);

__device__ __forceinline__ uint32_t t_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// shared-memory matrix descriptor, no swizzle: start address, leading-dimension and stride-dimension byte offsets
__device__ __forceinline__ uint64_t t_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void t_cp16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void t_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void t_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// bounded; gives up at once when another role of the CTA has given up; a wait that runs out raises the flag itself
__device__ __forceinline__ bool t_mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    const uint32_t addr = t_smem(bar);
    for (uint32_t it = 0; it < TC_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (ok) return true;
        if ((it & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void t_arrive(uint64_t *bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(t_smem(bar)) : "memory");
}
__device__ __forceinline__ void t_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void t_commit_mma(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(t_smem(bar)) : "memory");
}
// 32 consecutive columns of this thread's lane
__device__ __forceinline__ void t_ld32(float (&v)[32], uint32_t taddr) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
        "%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ uint32_t t_pack(float lo, float hi, float *sum) {
    const __half2 h = __floats2half2_rn(lo, hi);
    const float2 f = __half22float2(h);   // the row sum takes the weights as the second product sees them
    *sum += f.x + f.y;
    return *(const uint32_t *)&h;
}

__device__ __forceinline__ float t_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// profiling aid (B200_FA_PREFILL_PROFILE=1): SM clocks one thread of each role of CTA (0, 0) spends waiting at each of its
// barriers and working, summed over the tiles: [0..7] compute, [8..15] MMA lane, [16..19] K loader, [20..23] V loader
__device__ unsigned long long g_tc_prof[24];
#define TC_MARK(k)                                         \
    do {                                                   \
        if (prof) {                                        \
            const long long t_now = clock64();             \
            g_tc_prof[k] += (unsigned long long)(t_now - t_prev); \
            t_prev = t_now;                                \
        }                                                  \
    } while (0)

struct alignas(16) TcBars {
    uint64_t k_full[TC_NS], k_free[TC_NS], v_full[TC_NS], v_free[TC_NS], s_done[TC_NS], s_free[TC_NS], p_full[TC_NS], p_free[TC_NS];
    uint64_t o_done[2], pv_free[2], mx_done;
    uint32_t tmem_base;
    int abort_flag;
    int vis[2][8];           // tile j's verdict in vis[0][j % 8] | vis[1][j % 8] (one word per K loader warp): does any row of the CTA see anything in it
    float mx[2][2][TC_BM];   // [tile parity][half][row]: the two column halves of a row tell each other their maxima
    float lsum[2][TC_BM];    // ... and, at the end, their shares of the row sum
};

__global__ void __launch_bounds__(TC_THREADS, 1)
fa_prefill_tc_kernel(b200_flash_attn_args a, int group, float scale_log2, int *err, int profile) {
    extern __shared__ uint8_t tc_raw[];
    __shared__ TcBars bars;
    pdl_trigger();
    const uint32_t smem = (t_smem(tc_raw) + 1023u) & ~1023u;
    const uint32_t q_s = smem, k_s = q_s + TC_Q_BYTES, v_s = k_s + TC_NS * TC_K_BYTES, p_s = v_s + TC_NS * TC_K_BYTES, m_s = p_s + TC_NS * TC_P_BYTES;
    uint8_t *gen = tc_raw + (smem - t_smem(tc_raw));   // the same region through generic addresses
    uint8_t *m_gen = gen + TC_Q_BYTES + 2 * TC_NS * TC_K_BYTES + TC_NS * TC_P_BYTES;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = blockIdx.y;
    const int64_t rows_total = a.n_tok * group;
    const int64_t row0 = (int64_t)blockIdx.x * TC_BM;
    const int64_t tok0 = row0 / group;
    int64_t tok_last = (row0 + TC_BM - 1) / group;
    if (tok_last >= a.n_tok) tok_last = a.n_tok - 1;
    const int n_tok_blk = (int)(tok_last - tok0 + 1);
    const int64_t n_tiles = (a.n_kv + TC_BN - 1) / TC_BN;
    volatile int *abort_flag = &bars.abort_flag;
    const bool prof = profile && lane == 0 && (warp == 0 || warp >= TC_MMA_WARP) && blockIdx.x == 0 && blockIdx.y == 0;
    long long t_prev = prof ? clock64() : 0;

    if (tid == 0) {
        auto init = [](uint64_t *b, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(t_smem(b)), "r"(count) : "memory"); };
        for (int i = 0; i < TC_NS; i++) {
            init(&bars.k_full[i], 64); init(&bars.k_free[i], 1); init(&bars.v_full[i], 32); init(&bars.v_free[i], 1);
            init(&bars.s_done[i], 1); init(&bars.s_free[i], TC_COMPUTE_WARPS * 32); init(&bars.p_full[i], TC_COMPUTE_WARPS * 32); init(&bars.p_free[i], 1);
        }
        for (int i = 0; i < 2; i++) { init(&bars.o_done[i], 1); init(&bars.pv_free[i], TC_COMPUTE_WARPS * 32); }
        init(&bars.mx_done, TC_COMPUTE_WARPS * 32);
        bars.abort_flag = 0;
        for (int i = 0; i < 8; i++) bars.vis[0][i] = bars.vis[1][i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(t_smem(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();   // q, the cache rows of this step and the mask come from earlier kernels / copies
    // ---- Q: f32 rows -> f16 core matrices (row r, piece c at (r / 8) 2048 + c 128 + (r % 8) 16); rows past the end are zero
    for (int i = tid; i < TC_BM * 16; i += TC_THREADS) {
        const int r = (i & 7) | ((i >> 7) << 3), c = ((i >> 3) & 3) | (((i >> 5) & 3) << 2);   // 8 rows of one piece per quarter-warp: every bank once
        const int64_t row = row0 + r;
        uint4 out = make_uint4(0, 0, 0, 0);
        if (row < rows_total) {
            const int64_t t = row / group;
            const int h = hk * group + (int)(row % group);
            const float *q = (const float *)((const uint8_t *)a.q + t * a.q_nb1 + (int64_t)h * a.q_nb2) + c * 8;
            const float4 x = *(const float4 *)q, y = *(const float4 *)(q + 4);
            const __half2 h0 = __floats2half2_rn(x.x, x.y), h1 = __floats2half2_rn(x.z, x.w), h2 = __floats2half2_rn(y.x, y.y), h3 = __floats2half2_rn(y.z, y.w);
            out = make_uint4(*(const uint32_t *)&h0, *(const uint32_t *)&h1, *(const uint32_t *)&h2, *(const uint32_t *)&h3);
        }
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(q_s + (uint32_t)((r >> 3) * 2048 + c * 128 + (r & 7) * 16)), "r"(out.x), "r"(out.y),
                     "r"(out.z), "r"(out.w)
                     : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q was written through the generic proxy; the MMAs read it through the async one
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;

    if (warp < TC_COMPUTE_WARPS) {
        // ================= compute warps: softmax of tile j, then the fold of tile j - 1's p v =================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_REGS_COMPUTE));
        const int half = warp >> 2;                                    // which half of the columns of its row this thread takes
        const int rowi = (warp & 3) * 32 + lane;                       // the row within the CTA = the tensor-memory lane
        const uint32_t t_row = tmem + ((uint32_t)(32 * (warp & 3)) << 16);   // the 32 lanes a warp may read: its index modulo 4
        const int64_t row = row0 + rowi;
        const bool live = row < rows_total;
        const int tok_rel = live ? (int)(row / group - tok0) : 0;
        float o[TC_D / 2];   // this thread's half of the output row
#pragma unroll
        for (int i = 0; i < TC_D / 2; i++) o[i] = 0.0f;
        float m_run = -INFINITY, l_run = 0.0f;
        float alpha_1 = 0.0f, alpha_2 = 0.0f;   // the rescalings that go with the two p v products still in flight (tiles j - 1, j - 2)
        bool vis_1 = false, vis_2 = false, ok = true;
        // o = o * alpha + p v of tile t, once its MMAs have completed; frees the p v region for tile t + 2
        auto fold = [&](int64_t t, float alpha_t, bool vis_t) {
            ok = t_mbar_wait(&bars.o_done[t & 1], (uint32_t)(t >> 1) & 1u, abort_flag);
            TC_MARK(7);
            if (!ok) return;
            if (vis_t) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int q4 = 0; q4 < 2; q4++) {
                    float pv[32];
                    t_ld32(pv, t_row + TC_TMEM_PV + (uint32_t)((t & 1) * TC_D + half * 64 + q4 * 32));
#pragma unroll
                    for (int i = 0; i < 32; i++) o[q4 * 32 + i] = fmaf(o[q4 * 32 + i], alpha_t, pv[i]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            t_arrive(&bars.pv_free[t & 1]);
        };
        for (int64_t tile = 0; tile < n_tiles && ok; tile++) {
            const int b = (int)(tile % TC_NS);
            const uint32_t ph = (uint32_t)(tile / TC_NS) & 1u;
            TC_MARK(0);   // everything else (fold, loop overhead)
            if (!(ok = t_mbar_wait(&bars.k_full[b], ph, abort_flag))) break;    // the mask rows and the verdict
            TC_MARK(1);
            const bool vis = (*(volatile int *)&bars.vis[0][tile & 7] | *(volatile int *)&bars.vis[1][tile & 7]) != 0;
            if (!(ok = t_mbar_wait(&bars.s_done[b], ph, abort_flag))) break;
            TC_MARK(2);
            float alpha = 1.0f, sc[32], mx = -INFINITY;
            if (vis) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                t_ld32(sc, t_row + (uint32_t)(b * TC_BN + half * 32));
                const uint8_t *mrow = m_gen + b * TC_M_BYTES + tok_rel * TC_MPITCH + half * 64;
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const uint4 mv = *(const uint4 *)(mrow + c * 16);
                    const uint32_t w[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 mf = __half22float2(*(const __half2 *)&w[e]);
                        float *sv = &sc[c * 8 + e * 2];
                        sv[0] = live ? fmaf(sv[0], scale_log2, mf.x * TC_LOG2E) : -INFINITY;
                        sv[1] = live ? fmaf(sv[1], scale_log2, mf.y * TC_LOG2E) : -INFINITY;
                        mx = fmaxf(mx, fmaxf(sv[0], sv[1]));
                    }
                }
                bars.mx[tile & 1][half][rowi] = mx;
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            TC_MARK(3);   // ld S, scale, mask, max
            t_arrive(&bars.s_free[b]);      // this thread has read its part of the score region and of the mask rows
            t_arrive(&bars.mx_done);
            if (!(ok = t_mbar_wait(&bars.mx_done, (uint32_t)tile & 1u, abort_flag))) break;
            TC_MARK(4);
            if (!(ok = t_mbar_wait(&bars.p_free[b], ph ^ 1u, abort_flag))) break;   // p v of tile - 3 has read this P buffer
            TC_MARK(5);
            if (vis) {
                const float m_new = fmaxf(m_run, fmaxf(mx, bars.mx[tile & 1][half ^ 1][rowi]));
                // a row that has seen nothing yet keeps a zero accumulator; exp2(-inf - -inf) must not be formed
                alpha = m_run == -INFINITY ? 0.0f : t_ex2(m_run - m_new);
                const float sub = m_new == -INFINITY ? 0.0f : m_new;
                m_run = m_new;
                float psum = 0.0f;
                const uint32_t p_row = p_s + (uint32_t)(b * TC_P_BYTES + (rowi >> 3) * 1024 + (rowi & 7) * 16 + half * 512);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const float *sv = &sc[c * 8];
                    const uint32_t w0 = t_pack(t_ex2(sv[0] - sub), t_ex2(sv[1] - sub), &psum), w1 = t_pack(t_ex2(sv[2] - sub), t_ex2(sv[3] - sub), &psum);
                    const uint32_t w2 = t_pack(t_ex2(sv[4] - sub), t_ex2(sv[5] - sub), &psum), w3 = t_pack(t_ex2(sv[6] - sub), t_ex2(sv[7] - sub), &psum);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + c * 128), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
                l_run = fmaf(l_run, alpha, psum);   // this half's share of the row sum; both halves use the same maxima
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the weights, for the MMA's proxy
            }
            t_arrive(&bars.p_full[b]);
            TC_MARK(6);   // exp, P store
            // the p v product of two tiles ago has had two softmaxes to finish
            if (tile >= 2) fold(tile - 2, alpha_2, vis_2);
            alpha_2 = alpha_1; vis_2 = vis_1;
            alpha_1 = alpha; vis_1 = vis;
        }
        if (ok && n_tiles >= 2) fold(n_tiles - 2, alpha_2, vis_2);
        if (ok) fold(n_tiles - 1, alpha_1, vis_1);
        if (ok) {
            bars.lsum[half][rowi] = l_run;
            t_arrive(&bars.mx_done);
            ok = t_mbar_wait(&bars.mx_done, (uint32_t)n_tiles & 1u, abort_flag);
        }
        if (ok && live) {
            const float l = bars.lsum[0][rowi] + bars.lsum[1][rowi];   // the same order on both halves
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;   // a row that sees nothing gives zeros, as on the CPU
            float *dst = a.dst + ((row / group) * a.n_head + hk * group + row % group) * TC_D + half * (TC_D / 2);
#pragma unroll
            for (int i = 0; i < TC_D / 2; i += 4) *(float4 *)(dst + i) = make_float4(o[i] * inv, o[i + 1] * inv, o[i + 2] * inv, o[i + 3] * inv);
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_REGS_CONTROL));
        if (warp == TC_MMA_WARP) {
            // ================= the MMA lane: scores of tile j + 1 ahead of p v of tile j =================
            if (lane == 0) {
                bool ok = true;
                auto scores = [&](int64_t tile) {
                    const int b = (int)(tile % TC_NS);
                    const uint32_t ph = (uint32_t)(tile / TC_NS) & 1u;
                    TC_MARK(8);
                    if (!(ok = t_mbar_wait(&bars.k_full[b], ph, abort_flag))) return;
                    TC_MARK(9);
                    if (!(ok = t_mbar_wait(&bars.s_free[b], ph ^ 1u, abort_flag))) return;   // the softmax of tile - 3 has read this score region
                    TC_MARK(10);
                    if (*(volatile int *)&bars.vis[0][tile & 7] | *(volatile int *)&bars.vis[1][tile & 7]) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t kb = k_s + (uint32_t)(b * TC_K_BYTES);
#pragma unroll
                        for (int st = 0; st < TC_D / 16; st++)
                            t_mma(tmem + (uint32_t)(b * TC_BN), t_desc(q_s + st * 256, 128, 2048), t_desc(kb + st * 256, 128, 2048), TC_IDESC_S, st);
                        t_commit_mma(&bars.s_done[b]);
                        t_commit_mma(&bars.k_free[b]);
                    } else {
                        t_arrive(&bars.s_done[b]);
                        t_arrive(&bars.k_free[b]);
                    }
                };
                scores(0);
                if (ok && n_tiles > 1) scores(1);
                for (int64_t tile = 0; tile < n_tiles && ok; tile++) {
                    const int b = (int)(tile % TC_NS);
                    const uint32_t ph = (uint32_t)(tile / TC_NS) & 1u;
                    if (tile + 2 < n_tiles) scores(tile + 2);   // two tiles ahead of the p v product: the softmax never waits for scores
                    if (!ok) break;
                    TC_MARK(11);   // issuing the score MMAs
                    if (!(ok = t_mbar_wait(&bars.p_full[b], ph, abort_flag))) break;
                    TC_MARK(12);
                    if (!(ok = t_mbar_wait(&bars.v_full[b], ph, abort_flag))) break;
                    TC_MARK(13);
                    if (!(ok = t_mbar_wait(&bars.pv_free[tile & 1], ((uint32_t)(tile >> 1) & 1u) ^ 1u, abort_flag))) break;   // the fold of tile - 2 has read this p v region
                    TC_MARK(14);
                    if (*(volatile int *)&bars.vis[0][tile & 7] | *(volatile int *)&bars.vis[1][tile & 7]) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t pb = p_s + (uint32_t)(b * TC_P_BYTES), vb = v_s + (uint32_t)(b * TC_K_BYTES);
#pragma unroll
                        for (int j = 0; j < TC_BN / 16; j++)
                            t_mma(tmem + TC_TMEM_PV + (uint32_t)((tile & 1) * TC_D), t_desc(pb + j * 256, 128, 1024), t_desc(vb + j * 4096, 2048, 128), TC_IDESC_O, j);
                        t_commit_mma(&bars.o_done[tile & 1]);
                        t_commit_mma(&bars.v_free[b]);
                        t_commit_mma(&bars.p_free[b]);
                    } else {
                        t_arrive(&bars.o_done[tile & 1]);
                        t_arrive(&bars.v_free[b]);
                        t_arrive(&bars.p_free[b]);
                    }
                }
            }
        } else {
            // ================= the loaders: one warp for K tiles and mask rows, one for V tiles =================
            // core-matrix image of a tile of 64 cached rows (K-major for K, MN-major for V: the same bytes): piece c (16
            // bytes) of row p at (p / 8) 2048 + c 128 + (p % 8) 16.  Lanes 0-7 take 8 consecutive rows of one piece (8 x 16
            // bytes side by side in shared memory: every bank once per quarter-warp), lanes 8-15 the next piece of the same
            // rows, ...: the warp reads 64 contiguous bytes of each of 8 rows
            const bool is_k = warp != TC_VLOAD_WARP;
            const int part = warp == TC_KLOAD_WARP2 ? 1 : 0, parts = is_k ? 2 : 1;   // the K loaders take alternate groups of 32 pieces
            const uint8_t *base = is_k ? (const uint8_t *)a.k + (int64_t)hk * a.k_nb2 : (const uint8_t *)a.v + (int64_t)hk * a.v_nb2;
            const int64_t nb1 = is_k ? a.k_nb1 : a.v_nb1;
            auto stage_rows = [&](uint32_t dst, int64_t tile) {
#pragma unroll 4
                for (int i = lane + 32 * part; i < TC_BN * 16; i += 32 * parts) {
                    const int p = (i & 7) | ((i >> 7) << 3), c = ((i >> 3) & 3) | (((i >> 5) & 3) << 2);
                    int64_t pos = tile * TC_BN + p;
                    if (pos >= a.n_kv) pos = a.n_kv - 1;   // a ragged last tile re-reads the last row; its scores are masked
                    t_cp16(dst + (uint32_t)((p >> 3) * 2048 + c * 128 + (p & 7) * 16), base + pos * nb1 + c * 16);
                }
            };
            auto stage_mask = [&](int64_t tile) {
                const int buf = (int)(tile % TC_NS);
                const uint32_t dst0 = m_s + (uint32_t)(buf * TC_M_BYTES);
                uint8_t *gen0 = m_gen + buf * TC_M_BYTES;
                const bool whole = a.mask && (tile + 1) * TC_BN <= a.n_kv && (a.mask_nb1 % 16) == 0 && ((uintptr_t)a.mask % 16) == 0;
                for (int i = lane + 32 * part; i < n_tok_blk * 8; i += 64) {
                    const int t = i >> 3, c = i & 7;
                    if (whole) {
                        t_cp16(dst0 + (uint32_t)(t * TC_MPITCH + c * 16), (const uint8_t *)a.mask + (tok0 + t) * a.mask_nb1 + (tile * TC_BN) * 2 + c * 16);
                    } else {
                        uint16_t *d = (uint16_t *)(gen0 + t * TC_MPITCH + c * 16);
                        for (int e = 0; e < 8; e++) {
                            const int64_t pos = tile * TC_BN + c * 8 + e;
                            uint16_t v = 0;   // no mask tensor: everything inside the cache is visible
                            if (pos >= a.n_kv) v = 0xFC00;   // -inf past the end
                            else if (a.mask) v = *(const uint16_t *)((const uint8_t *)a.mask + (tok0 + t) * a.mask_nb1 + pos * 2);
                            d[e] = v;
                        }
                    }
                }
            };
            bool ok = true;
            if (is_k) {
                // tile j's copies are requested as soon as its buffer is free; tile j - 1's are then waited for, judged and published
                auto publish = [&](int64_t tile) {
                    const uint8_t *mt = m_gen + (int)(tile % TC_NS) * TC_M_BYTES;
                    int any = 0;
                    for (int i = lane + 32 * part; i < n_tok_blk * 8; i += 64) {   // the pieces this warp brought in
                        const uint4 v = *(const uint4 *)(mt + (i >> 3) * TC_MPITCH + (i & 7) * 16);
                        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int e = 0; e < 4; e++) any |= ((w[e] & 0xffffu) != 0xFC00u) | ((w[e] >> 16) != 0xFC00u);
                    }
                    any = __any_sync(0xffffffffu, any);
                    if (lane == 0) *(volatile int *)&bars.vis[part][tile & 7] = any;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the K rows, for the MMA's proxy
                    __syncwarp();
                    t_arrive(&bars.k_full[tile % TC_NS]);
                };
                for (int64_t tile = 0; tile < n_tiles && ok; tile++) {
                    TC_MARK(16);
                    // the buffer's previous tile (tile - 3): its score MMAs have read the K rows, its softmax the mask rows
                    if (!(ok = t_mbar_wait(&bars.k_free[tile % TC_NS], ((uint32_t)(tile / TC_NS) & 1u) ^ 1u, abort_flag))) break;
                    if (!(ok = t_mbar_wait(&bars.s_free[tile % TC_NS], ((uint32_t)(tile / TC_NS) & 1u) ^ 1u, abort_flag))) break;
                    TC_MARK(17);
                    stage_rows(k_s + (uint32_t)((tile % TC_NS) * TC_K_BYTES), tile);
                    stage_mask(tile);
                    t_commit();
                    TC_MARK(18);
                    if (tile > 0) {
                        t_wait<1>();
                        TC_MARK(19);
                        __syncwarp();
                        publish(tile - 1);
                    }
                }
                t_wait<0>();
                __syncwarp();
                if (ok) publish(n_tiles - 1);
            } else {
                int64_t pending = -1;   // the tile whose V copies are in flight
                for (int64_t tile = 0; tile < n_tiles && ok; tile++) {
                    const int b = (int)(tile % TC_NS);
                    const uint32_t ph = (uint32_t)(tile / TC_NS) & 1u;
                    TC_MARK(20);
                    if (!(ok = t_mbar_wait(&bars.k_full[b], ph, abort_flag))) break;          // the verdict
                    TC_MARK(21);
                    if (!(ok = t_mbar_wait(&bars.v_free[b], ph ^ 1u, abort_flag))) break;     // p v of tile - 3 has read this buffer
                    TC_MARK(22);
                    if (*(volatile int *)&bars.vis[0][tile & 7] | *(volatile int *)&bars.vis[1][tile & 7]) stage_rows(v_s + (uint32_t)(b * TC_K_BYTES), tile);
                    t_commit();
                    if (pending >= 0) {
                        t_wait<1>();
                        TC_MARK(23);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        t_arrive(&bars.v_full[pending % TC_NS]);
                    }
                    pending = tile;
                }
                t_wait<0>();
                if (ok && pending >= 0) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    t_arrive(&bars.v_full[pending % TC_NS]);
                }
            }
        }
    }
    // ---- teardown: every role has left its loop (finished, or gave up)
    asm volatile("cp.async.wait_all;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && bars.abort_flag) atomicExch(err, 4);
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace

// true: the tcgen05 prompt kernel took the call (*rc is its status); false: not a shape it handles
bool flash_attn_fast_prefill_tc(const b200_flash_attn_args *a, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (a->sinks || a->max_bias != 0.0f || a->logit_softcap != 0.0f || a->dk != TC_D || a->dv != TC_D || a->n_kv == 0 || a->n_tok == 0) return false;
    if (a->n_head % a->n_head_kv || a->n_head / a->n_head_kv < 2) return false;   // one head per KV head: 128 mask rows per CTA do not fit
    if (a->q_nb1 % 16 || a->q_nb2 % 16 || ((uintptr_t)a->q & 15) || ((uintptr_t)a->dst & 15)) return false;
    if (a->k_nb1 % 16 || a->v_nb1 % 16 || a->k_nb2 % 16 || a->v_nb2 % 16 || ((uintptr_t)a->k & 15) || ((uintptr_t)a->v & 15)) return false;
    if (a->mask && (a->mask_nb1 % 2 || ((uintptr_t)a->mask & 1))) return false;
    const int group = (int)(a->n_head / a->n_head_kv);
    const int64_t row_blocks = (a->n_tok * group + TC_BM - 1) / TC_BM;
    if (row_blocks > 0x7fffffffLL || a->n_head_kv > 65535) return false;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        *rc = cuda_fail(cudaGetLastError(), "flash_attn prefill: device query", __FILE__, __LINE__);
        return true;
    }
    static bool attr_done[64] = {};
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__); return true; }
        attr_done[dev] = true;
    }
    int *err = nullptr;
    *rc = device_error_word(&err);
    if (*rc != B200_STATUS_SUCCESS) return true;
    const char *pe = getenv("B200_FA_PREFILL_PROFILE");
    const int profile = (pe && pe[0] == '1') ? 1 : 0;
    if (profile) {
        static const unsigned long long zeros[24] = {0};
        cudaMemcpyToSymbolAsync(g_tc_prof, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice, s);
    }
    *rc = launch_pdl(fa_prefill_tc_kernel, dim3((unsigned)row_blocks, (unsigned)a->n_head_kv), dim3(TC_THREADS), (size_t)TC_SMEM, s, *a, group,
                     a->scale * TC_LOG2E, err, profile);
    return true;
}

// the clocks of the last profiled launch (see g_tc_prof)
int flash_attn_prefill_profile(unsigned long long *out, int n) {
    if (n > 24) n = 24;
    B200_CUDA(cudaMemcpyFromSymbol(out, g_tc_prof, (size_t)n * sizeof(unsigned long long)));
    return B200_STATUS_SUCCESS;
}

}  // namespace b200
