// FLASH_ATTN_EXT, fast mode, few query rows (single-token and small-batch decode): flash-decoding.
//
// The faithful kernels (flash_attn.cu) reproduce the CPU path's arithmetic bit for bit, including the f16
// accumulator that is rounded once per cached position: a dependent chain as long as the context.  This file is
// the mode for hosts that accept the tolerance asked of F16-KV attention (1e-3): the same function
//   softmax(q k^T * scale + mask) v        (crates/ggml/src/flash_attn.rs:482-736)
// with f32 accumulation and no ordered chain, so it can be cut freely:
//   * grid (splits, KV heads, row blocks): a CTA takes one KV head, a range of cached positions and up to 16 of the
//     query rows that read that KV head (the n_head / n_head_kv query heads of every token share the K / V tiles a
//     CTA stages: GQA head sharing), so the cache is read once per row block;
//   * K and V tiles of 32 positions are staged in shared memory with 16-byte cp.async copies (every cached row is
//     contiguous), double buffered; lane = position for the scores, lane = 4 value elements for P V;
//   * q stays in f32 (the CPU rounds it to f16 before its dot, flash_attn.rs:433), scores and P V accumulate in
//     f32, softmax runs online per row with exp2;
//   * every CTA leaves (max, sum, accumulator) per row; the last CTA of a (KV head, row block) to finish merges the
//     splits and writes the rows.
// Masked positions (-inf in the F16 mask) are skipped as the CPU skips them; a (row, tile) pair with nothing
// visible costs one mask read.  Not handled here (the caller falls back to the faithful kernels): sinks, ALiBi,
// softcap, dk != dv.
#include "common.cuh"
#include "flash_attn_fast.cuh"

namespace b200 {

namespace {

struct CtaSync {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

// partial[(((hk * row_blocks + rb) * n_splits + split) * FF_ROWS + r) * (D + 4)] = {acc[D], m, l, -, -}
template <int D, int NST, int ROWS>
__global__ void __launch_bounds__(FF_WARPS * 32)
fa_fast_rows_kernel(b200_flash_attn_args a, FastDims d, float scale_log2, float *__restrict__ partial, int *__restrict__ counters) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ FaFastMisc misc;
    __shared__ unsigned short vis_list[FF_MAX_LIST];   // several tokens per step: the tiles this unit's rows see anything in
    if (threadIdx.x == 0) misc.vis_list = vis_list;
    __syncthreads();
    pdl_trigger();
    pdl_wait();   // q, the cache rows of this step and the mask come from earlier kernels / copies
    fa_fast_unit<D, ROWS, NST>(a, d, scale_log2, partial, counters, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, (int)gridDim.z, (int)threadIdx.x, smem,
                    &misc, CtaSync());
}

int *g_fast_counters[64] = {nullptr};
__device__ int g_fast_counters_dev[4096];

}  // namespace

// How the cached positions are cut for `rows` query rows per unit on a device of `sms` SMs: enough units for two per
// SM, at least two tiles per unit once the context is long, at most FF_MAX_SPLITS per (KV head, row block).
// false: a shape the fast path does not take.
bool flash_attn_fast_dims(const b200_flash_attn_args *a, int sms, int rows, FastDims *out) {
    // units per SM the cut aims at: two; four for one token's rows over a long cache (a unit of 4 rows is small and there
    // are tiles enough to feed them: measured 68 -> 60 us at 32768 positions, while below 8192 the extra splits only
    // lengthen the merge)
    const int per_sm = rows <= 4 && a->n_kv > 8192 ? 4 : 2;
    FastDims d;
    d.T = (int)a->n_tok; d.H = (int)a->n_head; d.H_kv = (int)a->n_head_kv; d.group = d.H / d.H_kv;
    d.n_kv = a->n_kv;
    const int rows_total = d.T * d.group;
    const int row_blocks = (rows_total + rows - 1) / rows;
    if (d.H_kv > 65535 || row_blocks > 65535 || d.H_kv * row_blocks > 4096) return false;
    const int64_t n_tiles = (d.n_kv + FF_TILE - 1) / FF_TILE;
    int64_t want = (per_sm * (int64_t)sms + (int64_t)d.H_kv * row_blocks - 1) / ((int64_t)d.H_kv * row_blocks);
    if (want > FF_MAX_SPLITS) want = FF_MAX_SPLITS;
    if (want > n_tiles) want = n_tiles;
    if (want < 1) want = 1;
    d.tiles_per_split = (int)((n_tiles + want - 1) / want);
    d.n_splits = (int)((n_tiles + d.tiles_per_split - 1) / d.tiles_per_split);
    if (d.T > 1 && d.tiles_per_split > FF_MAX_LIST) return false;   // the visible-tile list of a unit is bounded
    *out = d;
    return true;
}

// true: the fast path took the call (*rc is its status); false: not a shape it handles
bool flash_attn_fast_rows(const b200_flash_attn_args *a, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (a->sinks || a->max_bias != 0.0f || a->logit_softcap != 0.0f || a->dk != a->dv || a->n_tok >= 64 || a->n_kv == 0 || a->n_tok == 0)
        return false;
    if (a->q_nb1 % 4 || a->q_nb2 % 4 || ((uintptr_t)a->dst & 15)) return false;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        *rc = cuda_fail(cudaGetLastError(), "flash_attn fast: device query", __FILE__, __LINE__);
        return true;
    }
    // Up to four query heads per KV head: a unit carries the rows of ONE token (4 rows, a quarter of the shared memory of a
    // 16-row unit).  With several tokens per step over a shared cache every token sees its own part of it, and a unit
    // that carries one token walks (and stages) only the tiles that token sees; 16-row units would stage every tile any
    // of four tokens sees and leave three quarters of their rows idle on it.
    const bool small = a->n_head / a->n_head_kv <= 4 && (a->n_tok == 1 || a->n_head / a->n_head_kv == 4);
    const int rows = small ? 4 : FF_ROWS;
    FastDims d;
    if (!flash_attn_fast_dims(a, sms, rows, &d)) return false;
    const int row_blocks = (d.T * d.group + rows - 1) / rows;
    if (!g_fast_counters[dev]) {   // a module variable: no allocation, zero-initialized on every device
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_fast_counters_dev);
        if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaGetSymbolAddress", __FILE__, __LINE__); return true; }
        g_fast_counters[dev] = (int *)p;
    }
    const int D = (int)a->dk;
    const size_t part_b = (size_t)d.H_kv * row_blocks * d.n_splits * rows * (D + 4) * 4;
    void *scratch = nullptr;
    *rc = scratch_get(part_b, &scratch);
    if (*rc != B200_STATUS_SUCCESS) return true;
    // a unit that walks several tiles keeps more of them in flight (long contexts: the cache comes from HBM); one or two
    // tiles per unit need no more than double buffering
    const bool deep = d.tiles_per_split >= 3;
    const dim3 grid((unsigned)d.n_splits, (unsigned)d.H_kv, (unsigned)row_blocks);
    const float scale_log2 = a->scale * LOG2E;
    float *part = (float *)scratch;
    int *cnt = g_fast_counters[dev];
    static bool attr_done[64] = {};
#define FA_FAST_CASE(DD, NN, RR)                                                                                                        \
    do {                                                                                                                                \
        const size_t smem = fa_fast_smem_bytes<DD, RR, NN>();                                                                           \
        if (!attr_done[dev]) {                                                                                                          \
            cudaError_t e = cudaSuccess;                                                                                                \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<128, 2, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<128, 16, 2>()); \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<128, 4, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<128, 16, 4>()); \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<64, 2, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<64, 16, 2>());   \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<64, 4, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<64, 16, 4>());   \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<128, 2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<128, 4, 2>());   \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<128, 3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<128, 4, 3>());   \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<64, 2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<64, 4, 2>());     \
            if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_fast_rows_kernel<64, 3, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_fast_smem_bytes<64, 4, 3>());     \
            if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__); return true; }                      \
            attr_done[dev] = true;                                                                                                      \
        }                                                                                                                               \
        *rc = launch_pdl(fa_fast_rows_kernel<DD, NN, RR>, grid, dim3(FF_WARPS * 32), smem, s, *a, d, scale_log2, part, cnt);               \
    } while (0)
    if (small) {
        if (D == 128) { if (deep) FA_FAST_CASE(128, 3, 4); else FA_FAST_CASE(128, 2, 4); }
        else { if (deep) FA_FAST_CASE(64, 3, 4); else FA_FAST_CASE(64, 2, 4); }
    } else {
        if (D == 128) { if (deep) FA_FAST_CASE(128, 4, 16); else FA_FAST_CASE(128, 2, 16); }
        else { if (deep) FA_FAST_CASE(64, 4, 16); else FA_FAST_CASE(64, 2, 16); }
    }
#undef FA_FAST_CASE
    return true;
}

}  // namespace b200
