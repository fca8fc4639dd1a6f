// FLASH_ATTN_EXT, fast mode, few query rows (single-token and small-batch decode), on the tensor cores: flash-decoding
// with mma.sync.
//
// The CUDA-core form (flash_attn_fast.cu) spends about 750 instructions per warp on a tile of 32 cached positions (a dot
// product per lane, a weighted sum per lane): it is bound by its own instruction stream, not by the cache traffic (2.2 TB/s
// at 32768 positions).  Here a block of 16 rows (the query heads of a KV head for up to 16 / group tokens; with one token
// and four heads per KV head four rows are live and the rest of the MMA tile is padding, which the tensor cores have to
// spare) multiplies a tile through mma.sync m16n8k16: about a tenth of the instructions per cached byte.
//   * grid (splits, KV heads, row blocks); a CTA of four warps stages tiles of 64 positions, double buffered (16-byte
//     cp.async pieces landing on a padded pitch, so that ldmatrix is free of bank conflicts; one bulk copy per cache row
//     against an mbarrier was measured too and was no quicker); the mask words a thread needs for the next tile are
//     fetched into registers one tile ahead; warp w takes positions 16 w .. 16 w + 15 of every tile:
//     q k^T as 16 MMAs (K through ldmatrix), online softmax over its 16 positions with its own running maximum and sum,
//     p v as 16 MMAs (V through ldmatrix.trans, p straight from the accumulator registers);
//   * at the end the four warps' (maximum, sum, accumulator) are merged in shared memory, the CTA leaves one partial per
//     row, and the last CTA of a (KV head, row block) merges the splits and writes the rows;
//   * with several tokens per step the CTA first lists the tiles of its range in which any of its rows sees anything and
//     stages only those.
// q is rounded to f16 as the CPU rounds it (crates/ggml/src/flash_attn.rs:433) and p to f16 for the second product:
// within 1e-3 of a float64 evaluation, like the prompt kernel.  Not handled (the caller falls back): sinks, ALiBi, softcap,
// dk != dv, more than 16 query heads per KV head.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int DM_BM = 16;            // rows per CTA (one MMA tile)
constexpr int DM_BN = 64;            // positions per staged tile (16 per warp)
constexpr int DM_WARPS = 4;
constexpr int DM_MAX_SPLITS = 64;
constexpr int DM_MAX_LIST = 1024;    // most tiles one CTA may walk when it first lists the visible ones
constexpr float DM_LOG2E = 1.4426950408889634f;

struct DmDims {
    int T, H, H_kv, group, row_blocks;
    int64_t n_kv;
    int n_splits, tiles_per_split;
    int strided;   // listed walk: split s takes tiles s, s + n_splits, .. instead of the range [s, s + 1) * tiles_per_split
};

__device__ __forceinline__ uint32_t d_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void d_cp16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d_smem(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void d_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void d_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void d_ldsm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void d_ldsm_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void d_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t d_pack(float lo, float hi, float *sum) {
    const __half2 h = __floats2half2_rn(lo, hi);
    const float2 f = __half22float2(h);   // the row sum takes the weights as the second product sees them
    *sum += f.x + f.y;
    return *(const uint32_t *)&h;
}

// partial[((hk * row_blocks + rb) * n_splits + split) * 16 + r][D + 4] = {acc[D], m, l, -, -}
// WIDE changes no code: the host gives that instance the largest shared-memory carve-out, for grids of more than two
// CTAs per SM
template <int D, bool WIDE>
__global__ void __launch_bounds__(DM_WARPS * 32, 3)
fa_decode_mma_kernel(b200_flash_attn_args a, DmDims d, float scale_log2, float *__restrict__ partial, int *__restrict__ counters) {
    constexpr int PITCH = D * 2 + 16;          // bytes per staged K / V row: the padding keeps ldmatrix rows on different banks
    constexpr int KS = D / 16, DB = D / 8, PSTRIDE = D + 4;
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *ks = smem;                                   // [2][DM_BN][PITCH]
    unsigned char *vs = ks + 2 * DM_BN * PITCH;                 // [2][DM_BN][PITCH]
    __shared__ unsigned short vis_list[DM_MAX_LIST];
    __shared__ int n_vis_s, is_last;
    __shared__ float wm[DM_WARPS][DM_BM], wl[DM_WARPS][DM_BM], lsum[DM_BM];

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int split = blockIdx.x, hk = blockIdx.y, rb = blockIdx.z;
    const int rows_total = d.T * d.group;
    const int row0 = rb * DM_BM;
    const int nrows = rows_total - row0 < DM_BM ? rows_total - row0 : DM_BM;
    const int tok0 = row0 / d.group;
    const int n_tok_blk = (row0 + nrows - 1) / d.group - tok0 + 1;
    const int64_t n_tiles_all = (d.n_kv + DM_BN - 1) / DM_BN;
    const int64_t tile0 = (int64_t)split * d.tiles_per_split;
    int64_t tile1 = tile0 + d.tiles_per_split;
    if (tile1 > n_tiles_all) tile1 = n_tiles_all;
    // thread t copies piece t % (D / 8) of rows t / (D / 8) + (1024 / D) j of K and of V
    constexpr int PIECES = D / 8, RSTEP = DM_WARPS * 32 / PIECES, PASSES = DM_BN / RSTEP;
    const int my_p = tid / PIECES, my_c = tid % PIECES;
    const unsigned char *kbase = (const unsigned char *)a.k + (int64_t)hk * a.k_nb2 + my_c * 16;
    const unsigned char *vbase = (const unsigned char *)a.v + (int64_t)hk * a.v_nb2 + my_c * 16;
    unsigned char *my_dst = ks + (size_t)my_p * PITCH + my_c * 16;

    auto stage = [&](int64_t tile, int buf) {
        {
            unsigned char *dk = my_dst + (size_t)buf * DM_BN * PITCH, *dv = dk + 2 * DM_BN * PITCH;
            const int64_t p0 = tile * DM_BN + my_p;
            if ((tile + 1) * DM_BN <= d.n_kv) {
                const unsigned char *sk = kbase + p0 * a.k_nb1, *sv = vbase + p0 * a.v_nb1;
#pragma unroll
                for (int j = 0; j < PASSES; j++) {
                    d_cp16(dk + (size_t)j * RSTEP * PITCH, sk + (int64_t)j * RSTEP * a.k_nb1);
                    d_cp16(dv + (size_t)j * RSTEP * PITCH, sv + (int64_t)j * RSTEP * a.v_nb1);
                }
            } else {
#pragma unroll
                for (int j = 0; j < PASSES; j++) {
                    int64_t pos = p0 + j * RSTEP;
                    if (pos >= d.n_kv) pos = d.n_kv - 1;
                    d_cp16(dk + (size_t)j * RSTEP * PITCH, kbase + pos * a.k_nb1);
                    d_cp16(dv + (size_t)j * RSTEP * PITCH, vbase + pos * a.v_nb1);
                }
            }
            d_commit();
        }
    };

    pdl_wait();   // q, the cache rows of this step and the mask come from earlier kernels / copies
    // this thread's rows of the block: lane / 4 and lane / 4 + 8
    const int r_a = lane >> 2, r_b = r_a + 8;
    const bool live_a = r_a < nrows, live_b = r_b < nrows;
    const int tok_a = live_a ? (row0 + r_a) / d.group - tok0 : 0, tok_b = live_b ? (row0 + r_b) / d.group - tok0 : 0;
    // the mask words of this thread's scores in a tile: [n][row a / row b], two positions each; -inf past the end of the cache
    const unsigned char *mrow_a = a.mask && live_a ? (const unsigned char *)a.mask + (int64_t)(tok0 + tok_a) * a.mask_nb1 : nullptr;
    const unsigned char *mrow_b = a.mask && live_b ? (const unsigned char *)a.mask + (int64_t)(tok0 + tok_b) * a.mask_nb1 : nullptr;
    const int pw = 16 * warp;   // this warp's positions of a tile
    auto mask_words = [&](int64_t tile, uint32_t (&mk)[2][2]) {
#pragma unroll
        for (int n = 0; n < 2; n++) {
            const int64_t pos = tile * DM_BN + pw + n * 8 + 2 * (lane & 3);
            uint32_t wa = 0, wb = 0;
            if (pos + 1 < d.n_kv) {
                if (mrow_a) wa = __ldg((const uint32_t *)(mrow_a + pos * 2));
                if (mrow_b) wb = __ldg((const uint32_t *)(mrow_b + pos * 2));
            } else if (pos < d.n_kv) {
                wa = 0xFC000000u | (mrow_a ? (uint32_t)__ldg((const uint16_t *)(mrow_a + pos * 2)) : 0u);
                wb = 0xFC000000u | (mrow_b ? (uint32_t)__ldg((const uint16_t *)(mrow_b + pos * 2)) : 0u);
            } else {
                wa = wb = 0xFC00FC00u;
            }
            mk[n][0] = wa; mk[n][1] = wb;
        }
    };
    // several tokens over a shared cache: the CTA first lists the tiles of its range in which any of its rows sees anything;
    // otherwise its first two tiles and the first tile's mask words are on their way while q is read
    const bool listed = a.mask != nullptr && d.T > 1;
    int n_walk = (int)(tile1 - tile0);
    const int64_t l_base = d.strided ? split : tile0, l_step = d.strided ? d.n_splits : 1;   // the listed walk's tiles: l_base + l_step i
    const int64_t n_local = !d.strided ? tile1 - tile0 : split < n_tiles_all ? (n_tiles_all - split + d.n_splits - 1) / d.n_splits : 0;
    uint32_t mk[2][2] = {{0u, 0u}, {0u, 0u}}, mk_next[2][2] = {{0u, 0u}, {0u, 0u}};
    if (!listed) {
        if (n_walk > 0) stage(tile0, 0); else d_commit();
        if (n_walk > 1) stage(tile0 + 1, 1); else d_commit();
        if (n_walk > 0) mask_words(tile0, mk);
    }
    uint32_t qf[KS][4];   // q as A fragments: {row a cols 16 s + 2 (lane % 4) .., row b same, row a cols + 8, row b cols + 8}
    {
        const int ha = hk * d.group + (live_a ? (row0 + r_a) % d.group : 0), hb = hk * d.group + (live_b ? (row0 + r_b) % d.group : 0);
        const float *qa = (const float *)((const unsigned char *)a.q + (int64_t)(tok0 + tok_a) * a.q_nb1 + (int64_t)ha * a.q_nb2);
        const float *qb = (const float *)((const unsigned char *)a.q + (int64_t)(tok0 + tok_b) * a.q_nb1 + (int64_t)hb * a.q_nb2);
        const int c0 = 2 * (lane & 3);
#pragma unroll
        for (int s = 0; s < KS; s++) {
            const float2 a0 = live_a ? __ldcg((const float2 *)(qa + 16 * s + c0)) : make_float2(0.f, 0.f);
            const float2 a1 = live_a ? __ldcg((const float2 *)(qa + 16 * s + c0 + 8)) : make_float2(0.f, 0.f);
            const float2 b0 = live_b ? __ldcg((const float2 *)(qb + 16 * s + c0)) : make_float2(0.f, 0.f);
            const float2 b1 = live_b ? __ldcg((const float2 *)(qb + 16 * s + c0 + 8)) : make_float2(0.f, 0.f);
            const __half2 h0 = __floats2half2_rn(a0.x, a0.y), h1 = __floats2half2_rn(b0.x, b0.y), h2 = __floats2half2_rn(a1.x, a1.y), h3 = __floats2half2_rn(b1.x, b1.y);
            qf[s][0] = *(const uint32_t *)&h0; qf[s][1] = *(const uint32_t *)&h1; qf[s][2] = *(const uint32_t *)&h2; qf[s][3] = *(const uint32_t *)&h3;
        }
    }
    float o[DB][4];
#pragma unroll
    for (int j = 0; j < DB; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;

    if (listed) {
        unsigned char *flags = smem;   // the staging area is not in use yet
        // with several tokens per step a split takes every n_splits-th tile, not a contiguous range: the tiles a row block sees
        // come in runs (a sequence's cells lie together), and contiguous ranges would leave some CTAs all of a run and others none
        // one warp per tile.  Aligned mask rows: lane = (token lane / 8, 16-byte piece lane % 8 of the tile's 128 mask bytes), so
        // four tokens' rows of a tile are one independent load per lane; otherwise lanes take two positions each, token by token
        const bool pieces = (((uintptr_t)a.mask | (uintptr_t)a.mask_nb1) & 15) == 0;
        for (int64_t tl = warp; tl < n_local; tl += DM_WARPS) {
            const int64_t tile = l_base + tl * l_step;
            bool any = false;
            if (pieces) {
                const int64_t p = tile * DM_BN + 8 * (lane & 7);
                for (int t = lane >> 3; t < n_tok_blk; t += 4) {
                    const unsigned char *mp = (const unsigned char *)a.mask + (int64_t)(tok0 + t) * a.mask_nb1 + p * 2;
                    if (p + 8 <= d.n_kv) {
                        const uint4 w = *(const uint4 *)mp;
                        any |= (w.x != 0xFC00FC00u) | (w.y != 0xFC00FC00u) | (w.z != 0xFC00FC00u) | (w.w != 0xFC00FC00u);
                    } else {
                        for (int e = 0; e < 8 && p + e < d.n_kv; e++) any |= *(const uint16_t *)(mp + 2 * e) != 0xFC00u;
                    }
                }
            } else {
                const int64_t p = tile * DM_BN + 2 * lane;
                for (int t = 0; t < n_tok_blk && !any; t++)
                    if (p < d.n_kv) {
                        const uint32_t two = p + 1 < d.n_kv ? *(const uint32_t *)((const unsigned char *)a.mask + (int64_t)(tok0 + t) * a.mask_nb1 + p * 2)
                                                            : (0xFC000000u | *(const uint16_t *)((const unsigned char *)a.mask + (int64_t)(tok0 + t) * a.mask_nb1 + p * 2));
                        any = ((two & 0xffffu) != 0xFC00u) | ((two >> 16) != 0xFC00u);
                    }
            }
            const unsigned hit = __ballot_sync(0xffffffffu, any);
            if (lane == 0) flags[tl] = hit != 0u;
        }
        __syncthreads();
        if (warp == 0) {   // ordered compaction, 32 tiles at a time
            int count = 0;
            for (int64_t base = 0; base < n_local; base += 32) {
                const bool f = base + lane < n_local && flags[base + lane];
                const unsigned bal = __ballot_sync(0xffffffffu, f);
                if (f) vis_list[count + __popc(bal & ((1u << lane) - 1u))] = (unsigned short)(base + lane);
                count += __popc(bal);
            }
            if (lane == 0) n_vis_s = count;
        }
        __syncthreads();
        n_walk = n_vis_s;
        if (n_walk > 0) stage(l_base + vis_list[0] * l_step, 0); else d_commit();
        if (n_walk > 1) stage(l_base + vis_list[1] * l_step, 1); else d_commit();
        if (n_walk > 0) mask_words(l_base + vis_list[0] * l_step, mk);
    }
    auto tile_at = [&](int i) -> int64_t { return listed ? l_base + vis_list[i] * l_step : tile0 + (int64_t)i; };

    // ldmatrix addressing (see flash_attn_prefill.cu): K non-transposed, V transposed
    const int k_row = (lane & 7) + ((lane >> 4) << 3), k_col = ((lane >> 3) & 1) * 16;
    const int v_row = (lane & 7) + (((lane >> 3) & 1) << 3), v_col = (lane >> 4) * 16;

    // two tiles in flight: tile it is waited for, multiplied, and its buffer handed to tile it + 2 (one commit group per
    // iteration, empty when there is no such tile, so that "all but the newest group" always means tile it)
    for (int it = 0; it < n_walk; it++) {
        const int buf = it & 1;
        d_wait_but_one();
        __syncthreads();   // the tile has landed for everyone
        if (it + 1 < n_walk) mask_words(tile_at(it + 1), mk_next);
        const unsigned char *kt = ks + (size_t)buf * DM_BN * PITCH, *vt = vs + (size_t)buf * DM_BN * PITCH;
        float s[2][4];
#pragma unroll
        for (int n = 0; n < 2; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
        for (int st = 0; st < KS; st++) {
            uint32_t b0, b1, b2, b3;
            d_ldsm_x4(b0, b1, b2, b3, kt + (size_t)(pw + k_row) * PITCH + st * 32 + k_col);
            d_mma(s[0], qf[st], b0, b1);
            d_mma(s[1], qf[st], b2, b3);
        }
        // scale, mask, the warp's row maxima
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < 2; n++) {
            const __half2 ha = *(const __half2 *)&mk[n][0], hb = *(const __half2 *)&mk[n][1];
            s[n][0] = live_a ? fmaf(s[n][0], scale_log2, __low2float(ha) * DM_LOG2E) : -INFINITY;
            s[n][1] = live_a ? fmaf(s[n][1], scale_log2, __high2float(ha) * DM_LOG2E) : -INFINITY;
            s[n][2] = live_b ? fmaf(s[n][2], scale_log2, __low2float(hb) * DM_LOG2E) : -INFINITY;
            s[n][3] = live_b ? fmaf(s[n][3], scale_log2, __high2float(hb) * DM_LOG2E) : -INFINITY;
            mx_a = fmaxf(mx_a, fmaxf(s[n][0], s[n][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[n][2], s[n][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        // nothing visible to any of the warp's rows among its 16 positions: nothing to add
        if (__ballot_sync(0xffffffffu, mx_a != -INFINITY || mx_b != -INFINITY) != 0u) {
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            // a row that has seen nothing yet keeps a zero accumulator; exp2(-inf - -inf) must not be formed
            const float al_a = m_a == -INFINITY ? 0.0f : exp2f(m_a - mn_a), al_b = m_b == -INFINITY ? 0.0f : exp2f(m_b - mn_b);
            const float sub_a = mn_a == -INFINITY ? 0.0f : mn_a, sub_b = mn_b == -INFINITY ? 0.0f : mn_b;
            const bool same = m_a == mn_a && m_b == mn_b;   // both factors are exactly 1, or the row's accumulator is still zero
            m_a = mn_a; m_b = mn_b;
            float ps_a = 0.0f, ps_b = 0.0f;
            uint32_t pf[4];   // p as the A fragment of the second product (k = the warp's 16 positions)
            pf[0] = d_pack(exp2f(s[0][0] - sub_a), exp2f(s[0][1] - sub_a), &ps_a);
            pf[1] = d_pack(exp2f(s[0][2] - sub_b), exp2f(s[0][3] - sub_b), &ps_b);
            pf[2] = d_pack(exp2f(s[1][0] - sub_a), exp2f(s[1][1] - sub_a), &ps_a);
            pf[3] = d_pack(exp2f(s[1][2] - sub_b), exp2f(s[1][3] - sub_b), &ps_b);
            l_a = fmaf(l_a, al_a, ps_a);
            l_b = fmaf(l_b, al_b, ps_b);
            if (!__all_sync(0xffffffffu, same)) {
#pragma unroll
                for (int j = 0; j < DB; j++) {
                    o[j][0] *= al_a; o[j][1] *= al_a; o[j][2] *= al_b; o[j][3] *= al_b;
                }
            }
#pragma unroll
            for (int e = 0; e < DB; e += 2) {
                uint32_t b0, b1, b2, b3;
                d_ldsm_x4_trans(b0, b1, b2, b3, vt + (size_t)(pw + v_row) * PITCH + e * 16 + v_col);
                d_mma(o[e], pf, b0, b1);
                d_mma(o[e + 1], pf, b2, b3);
            }
        }
        mk[0][0] = mk_next[0][0]; mk[0][1] = mk_next[0][1]; mk[1][0] = mk_next[1][0]; mk[1][1] = mk_next[1][1];
        __syncthreads();   // everyone is done with this buffer
        if (it + 2 < n_walk) stage(tile_at(it + 2), buf); else d_commit();
    }
    // ---- merge the four warps: row sums across the quad, then (maximum, sum) through shared memory, accumulators through
    // the K / V staging area
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    float *oacc = (float *)smem;   // [DM_WARPS][DM_BM][D] = 32 KB for D = 128 (the staging area is 68 KB); every copy into it has landed
    if ((lane & 3) == 0) {
        wm[warp][r_a] = m_a; wl[warp][r_a] = l_a;
        wm[warp][r_b] = m_b; wl[warp][r_b] = l_b;
    }
    {
        const int c0 = 2 * (lane & 3);
#pragma unroll
        for (int j = 0; j < DB; j++) {
            *(float2 *)(oacc + ((size_t)warp * DM_BM + r_a) * D + j * 8 + c0) = make_float2(o[j][0], o[j][1]);
            *(float2 *)(oacc + ((size_t)warp * DM_BM + r_b) * D + j * 8 + c0) = make_float2(o[j][2], o[j][3]);
        }
    }
    __syncthreads();
    float *mine = partial + (((int64_t)hk * d.row_blocks + rb) * d.n_splits + split) * DM_BM * PSTRIDE;
    for (int i = tid; i < nrows * (D / 4); i += DM_WARPS * 32) {
        const int r = i / (D / 4), e = 4 * (i % (D / 4));
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DM_WARPS; w++) M = fmaxf(M, wm[w][r]);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.0f;
#pragma unroll
        for (int w = 0; w < DM_WARPS; w++) {
            const float wgt = wm[w][r] == -INFINITY ? 0.0f : exp2f(wm[w][r] - M);
            const float4 v = *(const float4 *)(oacc + ((size_t)w * DM_BM + r) * D + e);
            acc.x = fmaf(v.x, wgt, acc.x); acc.y = fmaf(v.y, wgt, acc.y); acc.z = fmaf(v.z, wgt, acc.z); acc.w = fmaf(v.w, wgt, acc.w);
            L = fmaf(wl[w][r], wgt, L);
        }
        *(float4 *)(mine + (int64_t)r * PSTRIDE + e) = acc;
        if (e == 0) *(float2 *)(mine + (int64_t)r * PSTRIDE + D) = make_float2(M, L);
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(&counters[hk * d.row_blocks + rb], 1) == d.n_splits - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (tid == 0) counters[hk * d.row_blocks + rb] = 0;   // ready for the next launch
    // ---- the last CTA of the (KV head, row block) merges the splits
    const float *all = partial + ((int64_t)hk * d.row_blocks + rb) * d.n_splits * DM_BM * PSTRIDE;
    float *mw = (float *)smem;                      // [DM_BM][DM_MAX_SPLITS] maxima, then weights
    float *lw = mw + DM_BM * DM_MAX_SPLITS;         // [DM_BM][DM_MAX_SPLITS] sums
    for (int i = tid; i < nrows * d.n_splits; i += DM_WARPS * 32) {
        const int r = i / d.n_splits, sp = i - r * d.n_splits;
        const float2 ml = __ldcg((const float2 *)(all + ((int64_t)sp * DM_BM + r) * PSTRIDE + D));
        mw[r * DM_MAX_SPLITS + sp] = ml.x;
        lw[r * DM_MAX_SPLITS + sp] = ml.y;
    }
    __syncthreads();
    for (int r = warp; r < nrows; r += DM_WARPS) {   // DM_MAX_SPLITS = 64: two splits per lane
        const float m0 = lane < d.n_splits ? mw[r * DM_MAX_SPLITS + lane] : -INFINITY;
        const float m1 = lane + 32 < d.n_splits ? mw[r * DM_MAX_SPLITS + lane + 32] : -INFINITY;
        float M = fmaxf(m0, m1);
#pragma unroll
        for (int o_ = 16; o_ > 0; o_ >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o_));
        const float w0 = m0 == -INFINITY ? 0.0f : exp2f(m0 - M), w1 = m1 == -INFINITY ? 0.0f : exp2f(m1 - M);
        float L = 0.0f;
        if (lane < d.n_splits) { mw[r * DM_MAX_SPLITS + lane] = w0; L = lw[r * DM_MAX_SPLITS + lane] * w0; }
        if (lane + 32 < d.n_splits) { mw[r * DM_MAX_SPLITS + lane + 32] = w1; L = fmaf(lw[r * DM_MAX_SPLITS + lane + 32], w1, L); }
#pragma unroll
        for (int o_ = 16; o_ > 0; o_ >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o_);
        if (lane == 0) lsum[r] = L;
    }
    __syncthreads();
    // a thread's (row, four columns) items side by side, so that their loads of a split's partials are in flight together
    constexpr int ITEMS = DM_BM * (D / 4) / (DM_WARPS * 32);
    float4 acc[ITEMS];
#pragma unroll
    for (int it = 0; it < ITEMS; it++) acc[it] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
    for (int sp = 0; sp < d.n_splits; sp++) {
#pragma unroll
        for (int it = 0; it < ITEMS; it++) {
            const int i = tid + it * DM_WARPS * 32;
            if (i < nrows * (D / 4)) {
                const int r = i / (D / 4), e = 4 * (i - r * (D / 4));
                const float4 v = __ldcg((const float4 *)(all + ((int64_t)sp * DM_BM + r) * PSTRIDE + e));
                const float w = mw[r * DM_MAX_SPLITS + sp];
                acc[it].x = fmaf(v.x, w, acc[it].x); acc[it].y = fmaf(v.y, w, acc[it].y); acc[it].z = fmaf(v.z, w, acc[it].z); acc[it].w = fmaf(v.w, w, acc[it].w);
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; it++) {
        const int i = tid + it * DM_WARPS * 32;
        if (i < nrows * (D / 4)) {
            const int r = i / (D / 4), e = 4 * (i - r * (D / 4));
            const int row = row0 + r, t = row / d.group, h = hk * d.group + row % d.group;
            const float L = lsum[r];
            const float inv = L > 0.0f ? 1.0f / L : 0.0f;   // a row that sees nothing gives zeros, as on the CPU
            *(float4 *)(a.dst + ((int64_t)t * d.H + h) * D + e) = make_float4(acc[it].x * inv, acc[it].y * inv, acc[it].z * inv, acc[it].w * inv);
        }
    }
}

int *g_dm_counters[64] = {nullptr};
__device__ int g_dm_counters_dev[4096];

}  // namespace

// true: the tensor-core decode kernel took the call (*rc is its status); false: not a shape it handles
bool flash_attn_decode_mma(const b200_flash_attn_args *a, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (a->sinks || a->max_bias != 0.0f || a->logit_softcap != 0.0f || a->dk != a->dv || (a->dk != 64 && a->dk != 128) || a->n_tok >= 64 || a->n_kv == 0 ||
        a->n_tok == 0)
        return false;
    if (a->n_head % a->n_head_kv || a->n_head / a->n_head_kv > DM_BM || DM_BM % (a->n_head / a->n_head_kv)) return false;   // whole tokens per row block
    if (a->q_nb1 % 8 || a->q_nb2 % 8 || ((uintptr_t)a->q & 7) || ((uintptr_t)a->dst & 15)) return false;
    if (a->k_nb1 % 16 || a->v_nb1 % 16 || a->k_nb2 % 16 || a->v_nb2 % 16 || ((uintptr_t)a->k & 15) || ((uintptr_t)a->v & 15)) return false;
    if (a->mask && (a->mask_nb1 % 4 || ((uintptr_t)a->mask & 3))) return false;
    DmDims d;
    d.T = (int)a->n_tok; d.H = (int)a->n_head; d.H_kv = (int)a->n_head_kv; d.group = d.H / d.H_kv;
    d.n_kv = a->n_kv;
    d.row_blocks = (d.T * d.group + DM_BM - 1) / DM_BM;
    if (d.H_kv > 65535 || d.row_blocks > 65535 || d.H_kv * d.row_blocks > 4096) return false;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        *rc = cuda_fail(cudaGetLastError(), "flash_attn decode: device query", __FILE__, __LINE__);
        return true;
    }
    const int64_t n_tiles = (d.n_kv + DM_BN - 1) / DM_BN;
    // three CTAs per SM (what the shared memory allows), at most DM_MAX_SPLITS splits, at least one tile each
    // (rounded down: a grid of a few CTAs more than the SMs hold at once runs those few as a second wave and takes twice the time)
    int64_t want = 3 * (int64_t)sms / ((int64_t)d.H_kv * d.row_blocks);
    if (want > DM_MAX_SPLITS) want = DM_MAX_SPLITS;
    if (want > n_tiles) want = n_tiles;
    if (want < 1) want = 1;
    d.tiles_per_split = (int)((n_tiles + want - 1) / want);
    d.n_splits = (int)((n_tiles + d.tiles_per_split - 1) / d.tiles_per_split);
    if (d.T > 1 && d.tiles_per_split > DM_MAX_LIST) return false;
    {
        const char *e = getenv("B200_FA_DECODE_STRIDED");
        d.strided = !(e && e[0] == '0');   // on unless switched off
    }
    if (!g_dm_counters[dev]) {   // a module variable: no allocation, zero-initialized on every device
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_dm_counters_dev);
        if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetSymbolAddress", __FILE__, __LINE__); return true; }
        g_dm_counters[dev] = (int *)p;
    }
    const int D = (int)a->dk;
    const size_t part_b = (size_t)d.H_kv * d.row_blocks * d.n_splits * DM_BM * (D + 4) * 4;
    void *scratch = nullptr;
    *rc = scratch_get(part_b, &scratch);
    if (*rc != B200_STATUS_SUCCESS) return true;
    const size_t smem = (size_t)4 * DM_BN * (D * 2 + 16);
    // more than two CTAs per SM: the instance with the largest shared-memory carve-out (B200_FA_DECODE_WIDE=0 / 1 overrides,
    // read per call)
    bool wide = (int64_t)d.n_splits * d.H_kv * d.row_blocks > 2 * (int64_t)sms;
    if (const char *ev = getenv("B200_FA_DECODE_WIDE")) wide = ev[0] == '1';
    const dim3 grid((unsigned)d.n_splits, (unsigned)d.H_kv, (unsigned)d.row_blocks);
    const float scale_log2 = a->scale * DM_LOG2E;
#define DM_CASE(DD, BB)                                                                                                                              \
    do {                                                                                                                                             \
        static bool attr_done[64] = {};                                                                                                              \
        if (!attr_done[dev]) {                                                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(fa_decode_mma_kernel<DD, BB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * DM_BN * (DD * 2 + 16)); \
            if (e == cudaSuccess && BB)                                                                                                              \
                e = cudaFuncSetAttribute(fa_decode_mma_kernel<DD, BB>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared); \
            if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__); return true; }                                   \
            attr_done[dev] = true;                                                                                                                   \
        }                                                                                                                                            \
        *rc = launch_pdl(fa_decode_mma_kernel<DD, BB>, grid, dim3(DM_WARPS * 32), smem, s, *a, d, scale_log2, (float *)scratch, g_dm_counters[dev]); \
    } while (0)
    if (D == 128 && wide) DM_CASE(128, true);
    else if (D == 128) DM_CASE(128, false);
    else if (wide) DM_CASE(64, true);
    else DM_CASE(64, false);
#undef DM_CASE
    return true;
}

}  // namespace b200
