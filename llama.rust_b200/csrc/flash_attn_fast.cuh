// The unit of work of fast-mode attention over few query rows (flash-decoding), shared by the stand-alone kernel
// (flash_attn_fast.cu) and the persistent decode kernel (decode_persistent.cu).  See flash_attn_fast.cu for the method.
#pragma once
#include "common.cuh"

namespace b200 {


constexpr int FF_TILE = 32;          // positions per tile
constexpr int FF_ROWS = 16;          // query rows per CTA
constexpr int FF_WARPS = 4;
constexpr int FF_MAX_SPLITS = 64;
constexpr int FF_MAX_LIST = 2048;    // most tiles one CTA may walk when it first lists the visible ones
constexpr float LOG2E = 1.4426950408889634f;

struct FastDims {
    int T, H, H_kv, group;
    int64_t n_kv;
    int n_splits;
    int tiles_per_split;
};
// the cut of the cached positions into splits (flash_attn_fast.cu); false: a shape the fast path does not take
bool flash_attn_fast_dims(const b200_flash_attn_args *a, int sms, int rows, FastDims *out);

__device__ __forceinline__ void cp_async16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// partial[(((hk * row_blocks + rb) * n_splits + split) * FF_ROWS + r) * (D + 4)] = {acc[D], m, l, -, -}
// The work of one (split, KV head, row block) by a group of FF_WARPS warps: the whole CTA of fa_fast_rows_kernel, or
// four warps of a persistent kernel that walks such units.  sync() is a barrier over exactly those warps; smem is the
// group's own block of fa_fast_smem_bytes<D>(); misc its FaFastMisc.  Every group that runs the same unit on the same
// inputs produces the same bits: the arithmetic does not depend on who calls.
struct FaFastMisc {
    int is_last;
    int n_vis;
    float lsum[FF_ROWS];
    unsigned short *vis_list;   // [FF_MAX_LIST], only walked when several tokens share the step (null otherwise)
};
template <int D, int ROWS, int NST>
__host__ __device__ constexpr size_t fa_fast_smem_bytes() {
    return (size_t)2 * NST * FF_TILE * (D * 2 + 16) + (size_t)ROWS * D * 4 + (size_t)ROWS * FF_MAX_SPLITS * 4;
}
// ROWS: the most query rows a unit carries (a multiple of FF_WARPS); it sizes the group's shared memory and the
// partials' layout, not the arithmetic of a row.  NST: K / V tiles in flight or in use at a time (2 = double buffering;
// a unit that walks many tiles of a long context keeps HBM busier with more); it does not touch the arithmetic either.
template <int D, int ROWS, int NST, class Sync>
__device__ __forceinline__ void fa_fast_unit(const b200_flash_attn_args &a, const FastDims &d, float scale_log2, float *__restrict__ partial,
                                             int *__restrict__ counters, int split, int hk, int rb, int row_blocks, int tid,
                                             unsigned char *smem, FaFastMisc *misc, Sync sync) {
    constexpr int KSTRIDE = D * 2 + 16;                      // bytes per staged row: 16 bytes of padding keep lanes on different banks
    constexpr int VEC = D / 32;                              // value elements per lane
    unsigned char *ks = smem;                                // [NST][FF_TILE][KSTRIDE]
    unsigned char *vs = ks + NST * FF_TILE * KSTRIDE;        // [NST][FF_TILE][KSTRIDE]
    float *qs = (float *)(vs + NST * FF_TILE * KSTRIDE);     // [ROWS][D]
    float *ps = qs + ROWS * D;                            // [ROWS][FF_TILE]; the merge reuses it as [ROWS][FF_MAX_SPLITS]
    const int lane = tid & 31, warp = tid >> 5;
    const int rows_total = d.T * d.group;                    // rows that read this KV head: row = t * group + g
    const int row0 = rb * ROWS;
    const int nrows = rows_total - row0 < ROWS ? rows_total - row0 : ROWS;
    const int64_t tile0 = (int64_t)split * d.tiles_per_split;
    const int64_t n_tiles_all = (d.n_kv + FF_TILE - 1) / FF_TILE;
    int64_t tile1 = tile0 + d.tiles_per_split;
    if (tile1 > n_tiles_all) tile1 = n_tiles_all;
    const unsigned char *kbase = (const unsigned char *)a.k + (int64_t)hk * a.k_nb2;
    const unsigned char *vbase = (const unsigned char *)a.v + (int64_t)hk * a.v_nb2;

    for (int i = tid; i < nrows * D; i += FF_WARPS * 32) {
        const int r = row0 + i / D, e = i % D;
        const int t = r / d.group, h = hk * d.group + r % d.group;
        const float *q = (const float *)((const unsigned char *)a.q + (int64_t)t * a.q_nb1 + (int64_t)h * a.q_nb2);
        qs[i] = __ldcg(q + e);   // straight from L2: in a persistent kernel another SM wrote it a moment ago
    }

    auto stage = [&](int64_t tile, int buf) {
        // FF_TILE rows of D halves each for K and V: D / 8 16-byte pieces per row
        constexpr int PIECES = D / 8;
        for (int i = tid; i < FF_TILE * PIECES; i += FF_WARPS * 32) {
            const int p = i / PIECES, c = i % PIECES;
            int64_t pos = tile * FF_TILE + p;
            if (pos >= d.n_kv) pos = d.n_kv - 1;   // a ragged last tile re-reads the last row; its scores are masked below
            cp_async16(ks + ((size_t)buf * FF_TILE + p) * KSTRIDE + c * 16, kbase + pos * a.k_nb1 + c * 16);
            cp_async16(vs + ((size_t)buf * FF_TILE + p) * KSTRIDE + c * 16, vbase + pos * a.v_nb1 + c * 16);
        }
        cp_async_commit();
    };

    // per warp: rows warp, warp + 4, ...; per row the running max (in log2 units), sum and VEC accumulator elements per lane
    constexpr int RPW = ROWS / FF_WARPS;
    float m_run[RPW], l_run[RPW], acc[RPW][VEC];
#pragma unroll
    for (int i = 0; i < RPW; i++) {
        m_run[i] = -INFINITY;
        l_run[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < VEC; j++) acc[i][j] = 0.0f;
    }

    // Several tokens per step over a shared cache (batched decode): every row sees a small part of the cells.  The
    // CTA first lists the tiles of its range in which any of its rows sees anything (one mask read per row and
    // tile), and stages K / V for those only.
    unsigned short *vis_list = misc->vis_list;
    const bool listed = a.mask != nullptr && d.T > 1;
    int n_walk = (int)(tile1 - tile0);
    if (listed) {
        const int t_lo = row0 / d.group, t_hi = (row0 + nrows - 1) / d.group;
        unsigned char *flags = (unsigned char *)ps;   // [tiles of the range], ps is not in use yet
        for (int64_t tl = warp; tl < tile1 - tile0; tl += FF_WARPS) {
            const int64_t p = (tile0 + tl) * FF_TILE + lane;
            bool any = false;
            for (int t = t_lo; t <= t_hi && !any; t++)
                any = p < d.n_kv && __half2float(((const __half *)((const unsigned char *)a.mask + (int64_t)t * a.mask_nb1))[p]) != -INFINITY;
            const unsigned hit = __ballot_sync(0xffffffffu, any);
            if (lane == 0) flags[tl] = hit != 0u;
        }
        sync();
        if (warp == 0) {   // ordered compaction, 32 tiles at a time
            int count = 0;
            for (int64_t base = 0; base < tile1 - tile0; base += 32) {
                const bool f = base + lane < tile1 - tile0 && flags[base + lane];
                const unsigned bal = __ballot_sync(0xffffffffu, f);
                if (f) vis_list[count + __popc(bal & ((1u << lane) - 1u))] = (unsigned short)(base + lane);
                count += __popc(bal);
            }
            if (lane == 0) misc->n_vis = count;
        }
        sync();
        n_walk = misc->n_vis;
    }
    auto tile_at = [&](int i) -> int64_t { return tile0 + (listed ? (int64_t)vis_list[i] : (int64_t)i); };

    // NST - 1 tiles ahead of the one in use; a copy group is committed per step whether or not a tile was left to
    // stage, so that "all but the last NST - 2 groups have landed" always means "tile `it` has landed"
#pragma unroll
    for (int i = 0; i < NST - 1; i++) {
        if (i < n_walk) stage(tile_at(i), i);
        else cp_async_commit();
    }
    for (int it = 0; it < n_walk; it++) {
        const int64_t tile = tile_at(it);
        const int buf = it % NST;
        const int64_t pos = tile * FF_TILE + lane;
        // this tile's mask values travel while the K / V copies do: one round trip instead of two in a row
        float mvals[RPW];
#pragma unroll
        for (int i = 0; i < RPW; i++) {
            const int rl = warp + i * FF_WARPS;
            mvals[i] = 0.0f;
            if (rl < nrows && a.mask && pos < d.n_kv) {
                const int t = (row0 + rl) / d.group;
                mvals[i] = __half2float(((const __half *)((const unsigned char *)a.mask + (int64_t)t * a.mask_nb1))[pos]);
            }
        }
        // the buffer of tile it + NST - 1 is the one tile it - 1 used: free since the barrier that ended that step
        if (it + NST - 1 < n_walk) stage(tile_at(it + NST - 1), (it + NST - 1) % NST);
        else cp_async_commit();
        cp_async_wait<NST - 1>();
        sync();
        const unsigned char *krow = ks + ((size_t)buf * FF_TILE + lane) * KSTRIDE;
#pragma unroll
        for (int i = 0; i < RPW; i++) {
            const int rl = warp + i * FF_WARPS;        // row within the block
            if (rl >= nrows) break;
            // mask first: a hidden position is skipped, a row with nothing visible in this tile skips the tile
            const float mval = mvals[i];
            const bool visible = pos < d.n_kv && mval != -INFINITY;
            if (__ballot_sync(0xffffffffu, visible) == 0u) continue;
            float s = -INFINITY;
            if (visible) {
                const float *q = qs + rl * D;
                // four partial sums: one chain of D dependent multiply-adds would leave the warp waiting on its own results
                float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
                for (int c = 0; c < D / 8; c++) {
                    const uint4 kv = *(const uint4 *)(krow + c * 16);
                    const float4 q0 = *(const float4 *)(q + c * 8), q1 = *(const float4 *)(q + c * 8 + 4);
                    const float2 k0 = __half22float2(*(const __half2 *)&kv.x), k1 = __half22float2(*(const __half2 *)&kv.y);
                    const float2 k2 = __half22float2(*(const __half2 *)&kv.z), k3 = __half22float2(*(const __half2 *)&kv.w);
                    d0 = fmaf(q0.x, k0.x, d0); d1 = fmaf(q0.y, k0.y, d1); d2 = fmaf(q0.z, k1.x, d2); d3 = fmaf(q0.w, k1.y, d3);
                    d0 = fmaf(q1.x, k2.x, d0); d1 = fmaf(q1.y, k2.y, d1); d2 = fmaf(q1.z, k3.x, d2); d3 = fmaf(q1.w, k3.y, d3);
                }
                const float dot = (d0 + d1) + (d2 + d3);
                s = fmaf(dot, scale_log2, mval * LOG2E);   // log2 units: exp(x) = exp2(x * log2 e)
            }
            float tmax = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            const float m_new = fmaxf(m_run[i], tmax);
            const float alpha = m_run[i] == -INFINITY ? 0.0f : exp2f(m_run[i] - m_new);
            const float p = visible ? exp2f(s - m_new) : 0.0f;
            float psum = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l_run[i] = fmaf(l_run[i], alpha, psum);
            m_run[i] = m_new;
            ps[rl * FF_TILE + lane] = p;
            __syncwarp();
            // P V: lane owns value elements VEC * lane ..
            float o_[VEC];
#pragma unroll
            for (int j = 0; j < VEC; j++) o_[j] = acc[i][j] * alpha;
            const unsigned char *vcol = vs + (size_t)buf * FF_TILE * KSTRIDE + lane * VEC * 2;
#pragma unroll 8
            for (int pp = 0; pp < FF_TILE; pp++) {
                const float w = ps[rl * FF_TILE + pp];
                if (VEC == 4) {
                    const uint2 vv = *(const uint2 *)(vcol + (size_t)pp * KSTRIDE);
                    const float2 v0 = __half22float2(*(const __half2 *)&vv.x), v1 = __half22float2(*(const __half2 *)&vv.y);
                    o_[0] = fmaf(w, v0.x, o_[0]); o_[1] = fmaf(w, v0.y, o_[1]); o_[VEC - 2] = fmaf(w, v1.x, o_[VEC - 2]); o_[VEC - 1] = fmaf(w, v1.y, o_[VEC - 1]);
                } else {
                    const float2 v0 = __half22float2(*(const __half2 *)(vcol + (size_t)pp * KSTRIDE));
                    o_[0] = fmaf(w, v0.x, o_[0]); o_[VEC - 1] = fmaf(w, v0.y, o_[VEC - 1]);
                }
            }
#pragma unroll
            for (int j = 0; j < VEC; j++) acc[i][j] = o_[j];
            __syncwarp();
        }
        sync();   // the buffer staged two tiles ago is free again
    }

    // this CTA's partials
    constexpr int PSTRIDE = D + 4;
    float *mine = partial + (((int64_t)hk * row_blocks + rb) * d.n_splits + split) * ROWS * PSTRIDE;
#pragma unroll
    for (int i = 0; i < RPW; i++) {
        const int rl = warp + i * FF_WARPS;
        if (rl >= nrows) break;
        float *pr = mine + (int64_t)rl * PSTRIDE;
        if (lane == 0) { pr[D] = m_run[i]; pr[D + 1] = l_run[i]; }
#pragma unroll
        for (int j = 0; j < VEC; j++) pr[lane * VEC + j] = acc[i][j];
    }
    __threadfence();
    sync();
    if (tid == 0) misc->is_last = atomicAdd(&counters[hk * row_blocks + rb], 1) == d.n_splits - 1;
    sync();
    if (!misc->is_last) return;
    __threadfence();
    if (tid == 0) counters[hk * row_blocks + rb] = 0;   // ready for the next launch
    // merge the splits: a short serial tail on one CTA, so every step is laid out for few memory round trips.
    // (1) the (max, sum) pairs of every (row, split) come into shared memory with independent loads; (2) one warp per
    // row turns them into weights exp2(m - M) and the merged sum; (3) every thread sums four consecutive accumulator
    // elements of one row over the splits with 16-byte loads that do not depend on one another.
    const float *all = partial + ((int64_t)hk * row_blocks + rb) * d.n_splits * ROWS * PSTRIDE;
    float *mw = ps;                       // [ROWS][FF_MAX_SPLITS] maxima, then weights; ps is free now
    float *lw = qs;                       // [ROWS][FF_MAX_SPLITS] sums; qs is free too (ROWS * D >= ROWS * FF_MAX_SPLITS)
    float *lsum = misc->lsum;
    for (int i = tid; i < nrows * d.n_splits; i += FF_WARPS * 32) {
        const int rl = i / d.n_splits, sp = i - rl * d.n_splits;
        const float2 ml = __ldcg((const float2 *)(all + ((int64_t)sp * ROWS + rl) * PSTRIDE + D));
        mw[rl * FF_MAX_SPLITS + sp] = ml.x;
        lw[rl * FF_MAX_SPLITS + sp] = ml.y;
    }
    sync();
    for (int rl = warp; rl < nrows; rl += FF_WARPS) {   // FF_MAX_SPLITS = 64: two splits per lane
        const float m0 = lane < d.n_splits ? mw[rl * FF_MAX_SPLITS + lane] : -INFINITY;
        const float m1 = lane + 32 < d.n_splits ? mw[rl * FF_MAX_SPLITS + lane + 32] : -INFINITY;
        float M = fmaxf(m0, m1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float w0 = m0 == -INFINITY ? 0.0f : exp2f(m0 - M), w1 = m1 == -INFINITY ? 0.0f : exp2f(m1 - M);
        float L = 0.0f;
        if (lane < d.n_splits) { mw[rl * FF_MAX_SPLITS + lane] = w0; L = lw[rl * FF_MAX_SPLITS + lane] * w0; }
        if (lane + 32 < d.n_splits) { mw[rl * FF_MAX_SPLITS + lane + 32] = w1; L = fmaf(lw[rl * FF_MAX_SPLITS + lane + 32], w1, L); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
        if (lane == 0) lsum[rl] = L;
    }
    sync();
    for (int i = tid; i < nrows * (D / 4); i += FF_WARPS * 32) {
        const int rl = i / (D / 4), e = 4 * (i - rl * (D / 4));
        const float *pr = all + (int64_t)rl * PSTRIDE + e;
        float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
        for (int sp = 0; sp < d.n_splits; sp++) {
            const float4 v = __ldcg((const float4 *)(pr + (int64_t)sp * ROWS * PSTRIDE));
            const float w = mw[rl * FF_MAX_SPLITS + sp];
            o.x = fmaf(v.x, w, o.x); o.y = fmaf(v.y, w, o.y); o.z = fmaf(v.z, w, o.z); o.w = fmaf(v.w, w, o.w);
        }
        const int r = row0 + rl, t = r / d.group, h = hk * d.group + r % d.group;
        const float L = lsum[rl];
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;   // a row that sees nothing gives zeros, as on the CPU
        *(float4 *)(a.dst + ((int64_t)t * d.H + h) * D + e) = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
    }
}


}  // namespace b200
