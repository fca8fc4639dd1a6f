// One-token decode step of a llama-architecture graph as ONE persistent kernel (decode_persistent.cu).
//
// The host (backend.cu) recognizes the node list of a single-token step and describes it as a list of phases; the
// kernel's CTAs (one per SM) walk the phases with a grid-wide barrier between them.
#pragma once
#include "common.cuh"
#include "flash_attn_fast.cuh"

namespace b200 {

constexpr int DP_MAX_MATS = 3;
enum { DP_GEMV = 0, DP_ATTN = 1 };
enum { DP_PRO_PLAIN = 1, DP_PRO_NORM = 2 };
// what happens to the 32 outputs of a finished row tile
enum {
    DP_EPI_STORE = 0,       // dst[row] = v
    DP_EPI_ADD = 1,         // dst[row] = v; sum[row] = v + addend[row]        (the residual ADD after attn_output / ffn_down)
    DP_EPI_ROPE = 2,        // dst_raw[row] = v; dst[row] = rope(v)            (Q)
    DP_EPI_ROPE_CACHE = 3,  // the same, and the F16 rounding of rope(v) into the cache row of this step (K)
    DP_EPI_CACHE = 4,       // dst[row] = v and its F16 rounding into the cache row (V)
};

struct DpMat {
    const uint8_t *tiles;   // 32-row tile layout (weights.cu)
    float *dst;
    float *dst_raw;         // ROPE kinds only, may be null
    __half *cache;          // *_CACHE kinds: cell 0 of the layer's cache
    int type;               // B200_TYPE_Q4_K or B200_TYPE_Q6_K
    int n_tiles;
    int epi;
    int pad_;
};

struct DpPhase {
    int kind;
    // ---- DP_GEMV: quantize a row once per CTA, then row tiles of up to three matrices against it
    int n_mat;
    int pair;               // 1: job t = row tile t of mat[0] then of mat[1]; h_out[row] = silu(mat0 row) * (mat1 row)
    int prologue;           // DP_PRO_PLAIN: the row as it is; DP_PRO_NORM: (x * rms_scale(x)) * norm_w
    int k, nb;              // row length, 256-element groups
    int jobs;               // row-tile jobs of the phase (pair: tiles of mat[0])
    int rot;                // rotation of the job -> CTA map, so that the odd tiles of consecutive phases land on different SMs
    float eps;
    int wide_end;           // pair: elements below this index take the 16-lane polynomial exp, the rest libm's
    int head_dim, n_dims;   // ROPE
    const float *x;
    const float *norm_w;
    float *y, *y_mul;       // DP_PRO_NORM: the norm and the weighted norm, written by one CTA (either may be null)
    const float *addend;    // DP_EPI_ADD
    float *sum;
    const float *rope_table;   // (cos, sin) pairs, one row of head_dim floats per position
    const int32_t *pos;        // this step's position (device)
    const int64_t *cell;       // this step's cache cell (device)
    int64_t rope_rows, cache_stride, cache_rows;   // cache_stride: elements per cell
    float *h_out;
    float *raw0, *raw1;     // pair: the two mat-muls' own outputs, may be null
    float *silu_out;        // pair: silu(mat0 row), may be null
    DpMat mat[DP_MAX_MATS];
    // ---- DP_ATTN: fast-mode attention of the step's one token (flash_attn_fast.cuh), rows = the query heads of a KV head
    b200_flash_attn_args fa;
    FastDims fd;
    float scale_log2;
    float *partial;
    int *counters;
};

// device words the kernel synchronizes on: zeroed (stream-ordered) before every launch
constexpr int DP_MAX_KV_HEADS = 254;
constexpr int DP_MAX_TIMED = 512;
constexpr int DP_TRACE_MAX = 4096;
struct DpSync {
    unsigned arrived;       // grid barrier arrivals, monotonic over the launch
    int abort;              // a CTA gave up a wait: everybody leaves
    int fa_counters[DP_MAX_KV_HEADS];   // attention: splits finished per KV head (the last one merges)
    unsigned long long t_phase[DP_MAX_TIMED];   // %globaltimer of CTA 0 at the start and after every grid barrier (profiling aid)
    unsigned long long t_first[DP_MAX_TIMED];   // earliest and latest arrival of a CTA at each grid barrier (only while profiling is on)
    unsigned long long t_last[DP_MAX_TIMED];
    unsigned long long trace[DP_TRACE_MAX];     // (event code << 56) | SM clock of one CTA's warp 0 (only while profiling is on)
    unsigned trace_n;
};

size_t decode_persistent_attn_partial_bytes(int n_head_kv, int n_splits, int head_dim);
size_t decode_persistent_work_bytes(int k);     // shared memory a mat-mul phase over rows of k elements needs ...
size_t decode_persistent_work_limit();          // ... and what the kernel has
int decode_persistent_norm_max_k();             // longest row a NORM prologue takes
int launch_decode_persistent(const DpPhase *dev_phases, int n_phases, DpSync *dev_sync, cudaStream_t s);

}  // namespace b200
