// Shared declarations of libggml-b200: status handling, device helpers, the
// device-side tile geometry of quantized tensors and the activation buffers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "ggml_b200.h"

namespace b200 {

// ---- status / error text ---------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what, const char *file, int line);

#define B200_CUDA(call)                                                        \
    do {                                                                       \
        cudaError_t e__ = (call);                                              \
        if (e__ != cudaSuccess) return b200::cuda_fail(e__, #call, __FILE__, __LINE__); \
    } while (0)

#define B200_REQUIRE(cond, ...)                                                \
    do {                                                                       \
        if (!(cond)) {                                                         \
            b200::set_error(__VA_ARGS__);                                      \
            return B200_STATUS_BACKEND_ERROR;                                  \
        }                                                                      \
    } while (0)

// ---- tile geometry ---------------------------------------------------------
// A quantized tensor of n_rows x k lives on the device as
//   [row tile of 32 rows][group of 256 k-elements][region][sub-chunk][row][unit bytes]
// so that lane r of a warp owns row r of the tile and every warp-wide load is
// one contiguous 512-byte (16 B per lane) access.  The bytes are those of the
// ggml blocks, only re-ordered; rows past n_rows in the last tile are zero.
constexpr int TILE_ROWS = 32;
constexpr int GROUP_K = 256;

struct TileGeom {
    int group_src_bytes;   // bytes of one row's 256-element group in ggml order
    int chunk_bytes;       // bytes of one (tile, group) chunk = 32 * group_src_bytes
};

__host__ __device__ inline int group_src_bytes(int type) {
    switch (type) {
        case B200_TYPE_Q4_K: return 144;
        case B200_TYPE_Q6_K: return 210;
        case B200_TYPE_Q8_0: return 8 * 34;
        case B200_TYPE_Q4_0: return 8 * 18;
        case B200_TYPE_MXFP4: return 8 * 17;
        default: return 0;
    }
}
__host__ __device__ inline int chunk_bytes(int type) { return TILE_ROWS * group_src_bytes(type); }

// Map byte p of a (tile, group) chunk to (row in tile, byte offset inside that
// row's 256-element group in ggml block order).  Regions per type:
//   Q4_K : [hdr 1x32x16][qs 8x32x16]           hdr = d, dmin, scales[12]
//   Q6_K : [ql 8x32x16][qh 4x32x16][sc 1x32x16][d 1x32x2]
//   Q8_0 : [qs 16x32x16][d 1x32x16]            sub s = block s/2, half s%2
//   Q4_0 : [qs 8x32x16][d 1x32x16]             sub s = block s
//   MXFP4: [qs 8x32x16][e 1x32x8]
__host__ __device__ inline void chunk_byte_to_src(int type, int p, int *row, int *src) {
    switch (type) {
        case B200_TYPE_Q4_K: {
            if (p < 512) { *row = p / 16; *src = p % 16; return; }
            int q = p - 512, sub = q / 512, r = (q % 512) / 16, b = q % 16;
            *row = r; *src = 16 + 16 * sub + b; return;
        }
        case B200_TYPE_Q6_K: {
            if (p < 4096) { int sub = p / 512, r = (p % 512) / 16, b = p % 16; *row = r; *src = 16 * sub + b; return; }
            if (p < 6144) { int q = p - 4096, sub = q / 512, r = (q % 512) / 16, b = q % 16; *row = r; *src = 128 + 16 * sub + b; return; }
            if (p < 6656) { int q = p - 6144; *row = q / 16; *src = 192 + q % 16; return; }
            { int q = p - 6656; *row = q / 2; *src = 208 + q % 2; return; }
        }
        case B200_TYPE_Q8_0: {
            if (p < 8192) { int sub = p / 512, r = (p % 512) / 16, b = p % 16; *row = r; *src = 34 * (sub / 2) + 2 + 16 * (sub % 2) + b; return; }
            { int q = p - 8192, r = q / 16, i = q % 16; *row = r; *src = 34 * (i / 2) + (i % 2); return; }
        }
        case B200_TYPE_Q4_0: {
            if (p < 4096) { int sub = p / 512, r = (p % 512) / 16, b = p % 16; *row = r; *src = 18 * sub + 2 + b; return; }
            { int q = p - 4096, r = q / 16, i = q % 16; *row = r; *src = 18 * (i / 2) + (i % 2); return; }
        }
        case B200_TYPE_MXFP4: {
            if (p < 4096) { int sub = p / 512, r = (p % 512) / 16, b = p % 16; *row = r; *src = 17 * sub + 1 + b; return; }
            { int q = p - 4096, r = q / 8, i = q % 8; *row = r; *src = 17 * i; return; }
        }
        default: *row = 0; *src = 0; return;
    }
}

inline bool is_quant_type(int type) { return group_src_bytes(type) != 0; }
inline bool is_k_quant(int type) { return type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K; }

// ---- quantized activations on the device -----------------------------------
// Structure of arrays; one instance holds m rows of k elements.
//   Q8_K kinds (A2, A3): qs[m][k] i8, d[m][k/256] f32, bsums[m][k/16] i16
//   Q8_0 (A1)          : qs[m][k] i8, dh[m][k/32] f16 bits (as the CPU stores them)
struct ActView {
    const int8_t *qs;
    const float *d;        // Q8_K scales
    const int16_t *bsums;  // Q8_K 16-element sums
    const uint16_t *dh;    // Q8_0 scales (f16 bits)
    int64_t k;
    // decode mat-muls (one activation row) may also emit result + addend: the residual ADD that follows
    // attn_output and ffn_down in a decoder layer (crates/llama/src/graph_arch.rs:209,226), one rounded add
    const float *addend = nullptr;
    float *sum = nullptr;
    // the few-rows kernels (8 to 31 activation rows) do the same for every row c: sum[c * ld_sum + i] = dst[c * lddst + i] + addend[c * ld_addend + i]
    int64_t ld_addend = 0, ld_sum = 0;
};
struct ActBuf {
    int8_t *qs;
    float *d;
    int16_t *bsums;
    uint16_t *dh;
    int64_t k;
    ActView view() const {
        ActView v;
        v.qs = qs; v.d = d; v.bsums = bsums; v.dh = dh; v.k = k;
        return v;
    }
};
// The f32 op in front of a one-row mat-mul, run inside the mat-mul's CTAs together with the Q8_K quantization of its
// result (see gemv_q4_K_row_kernel).
enum { ACT_PRO_NONE = 0, ACT_PRO_PLAIN = 1, ACT_PRO_NORM = 2, ACT_PRO_SILU = 3 };
struct ActPrologue {
    int mode = ACT_PRO_NONE;
    const float *x = nullptr;     // PLAIN, NORM: the row; SILU: the row silu is applied to
    const float *w = nullptr;     // NORM: the norm weight; SILU: the row the result is multiplied by
    float eps = 0.0f;             // NORM
    int wide_end = 0;             // SILU: elements below this index take the 16-lane polynomial exp, the rest libm's
    float *y = nullptr;           // NORM: x * rms_scale; SILU: silu(x) (either may be null)
    float *y_mul = nullptr;       // NORM: y * w; SILU: silu(x) * w
    ActBuf act_out = {nullptr, nullptr, nullptr, nullptr, 0};   // the quantized row, for later kernels (qs null: not wanted)
};
size_t act_scratch_bytes(int64_t m, int64_t k);
ActBuf act_carve(void *scratch, int64_t m, int64_t k);

// ---- kernels' host launchers (each returns a b200_status) -------------------
int launch_quantize_acts(int kind, int64_t m, int64_t k, const float *x, int64_t ldx, ActBuf out, cudaStream_t s);
int launch_repack(int type, int64_t n_rows, int64_t k, const uint8_t *src_blocks, uint8_t *tiles, bool inverse,
                  cudaStream_t s);
int launch_dequantize(int type, int64_t n_rows, int64_t k, const uint8_t *tiles, float *out, cudaStream_t s);
int launch_gemv(int type, int route, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts,
                float *dst, int64_t lddst, cudaStream_t s);

int launch_gemm_mma(int mode, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                    cudaStream_t s);
int launch_gemm_small_multi(int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                            const int64_t *lddst, cudaStream_t s);
bool gemm_small_multi_enabled();
int launch_gemm_rows_ring(int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                          const int64_t *lddst, cudaStream_t s);
void gemm_rows_ring_debug_wait(int spin_limit, int skip_unit);
bool gemv_rows_add_fusable(int type, int route, int64_t m);
int launch_gemm_tcgen05(int mode, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                        cudaStream_t s);
// Q8_0 / Q4_0 / MXFP4 / Q6_K prompt mat-muls on tcgen05 kind::i8 (gemm_tcgen05_i8.cu)
int launch_gemm_tcgen05_i8(int type, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                           cudaStream_t s);
// MUL_MAT_ID with the pairs grouped by expert on the device (MXFP4 / Q4_0 experts on the 8x8 route): gemm_tcgen05_i8.cu
size_t mmid_grouped_scratch_bytes(int64_t n_expert, int64_t n_pairs);
int launch_mul_mat_id_grouped(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok, int64_t n_ids, const uint8_t *tiles,
                              ActView acts, const int32_t *ids, float *dst, void *lists, cudaStream_t s);
// which Q4_K gemm-chain prompt kernel the time model prefers on a GPU of sm_count SMs: 0 integer, 3 / 4 two-pass with 64 / 128 columns
int gemm_chain_pick_for(int64_t n, int64_t m, int sm_count);
// Q4_K gemm chain with the scales folded into f16 operands, 128 x 64 per CTA (gemm_tcgen05_f16.cu)
int launch_gemm_tcgen05_f16x64(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s);
// the same chain in two passes: operands expanded to f16 images once, then a mat-mul that only copies, multiplies and drains (gemm_tcgen05_img.cu)
constexpr int GEMM_FAST_MIN_COLS = 64;   // activation rows from which the fast-numerics Q4_K prompt kernel takes the mat-mul
int gemm_tcgen05_f16_choice();   // gemm_tcgen05.cu: B200_GEMM_TCGEN05_F16 (-1 = unset: the library picks)
int launch_gemv_rows_multi(int type, int route, int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                           const int64_t *lddst, cudaStream_t s);   // gemv.cu
int launch_gemm_kq_fast_multi(int type, int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                              const int64_t *lddst, cudaStream_t s);   // up to three matrices over the same activations
int launch_gemm_kq_fast(int type, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s);   // Q4_K / Q6_K
int launch_gemm_q4_K_fast(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s);   // gemm_tcgen05_fast.cu
int launch_gemm_tcgen05_img(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s);
int launch_gemm_tcgen05_img128(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s);   // 128 activation rows per CTA
// up to four ROPE / SET_ROWS (F32 -> F16) nodes for one launch, see glue_batch_kernel
constexpr int GLUE_BATCH_MAX = 4;
enum { GLUE_ROPE = 1, GLUE_SET_ROWS = 2 };
struct GlueOp {
    int kind;
    int ne0;                 // ROPE: head size; SET_ROWS: row length
    int n_head, n_dims, neox;
    int64_t total;           // ROPE: tokens x heads x ne0 / 2 channel pairs; SET_ROWS: rows x ne0 elements
    const float *x;          // source
    int64_t x_nb1, x_nb2;    // ROPE: byte strides of head and token; SET_ROWS: x_nb1 = row stride in elements
    float *y;                // ROPE result
    int64_t y_nb1, y_nb2;
    const float *table;      // ROPE (cos, sin) table, one row per position (rows != null) or per token
    const int32_t *rows;
    int64_t n_rows;
    void *cache;            // SET_ROWS destination; ROPE: optional F16 rows that receive the rounded result
    int64_t cache_stride, cache_rows;
    const int64_t *cache_idx;
};
struct GlueBatch {
    GlueOp op[GLUE_BATCH_MAX];
    int count;
};
int launch_glue_batch(const GlueBatch &b, cudaStream_t s);
int launch_gemv_q4_K_multi(int count, const int64_t *n, const uint8_t *const *tiles, float *const *dst, int64_t k, ActView acts,
                           cudaStream_t s);
int launch_gemv_q4_K_row_fused(int count, const int64_t *n, const uint8_t *const *tiles, float *const *dst, int64_t k, ActView acts,
                               const ActPrologue &pro, cudaStream_t s);
int launch_gemv_q4_K_stream(int64_t n, int64_t k, const uint8_t *tiles, ActView acts, float *dst, cudaStream_t s);
int gemv_stream_error(int *code);
int device_error_word(int **flag);
int launch_get_rows_tiled(int type, int64_t table_rows, int64_t k, const uint8_t *tiles, const int32_t *ids, int64_t n,
                          float *out, int64_t out_stride, int *err, cudaStream_t s);
int launch_mul_mat_id(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok, int64_t n_ids,
                      const uint8_t *tiles, ActView acts, const int32_t *ids, float *dst, int *counts, cudaStream_t s);

// glue ops (glue_ops.cu); strides in elements unless the name says nb (bytes)
int launch_rms_norm(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *w, float *y_mul,
                    int64_t y_mul_stride, int64_t ne0, int64_t nrows, float eps, cudaStream_t s);
int launch_rms_norm_q8(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *w, float *y_mul,
                       int64_t y_mul_stride, int64_t ne0, int64_t nrows, float eps, ActBuf act, int64_t m4, cudaStream_t s);
int launch_silu_q8(const float *x, int64_t x_stride, const float *g, int64_t g_stride, float *y, int64_t y_stride, float *y_mul,
                   int64_t y_mul_stride, int64_t ne0, int64_t nrows, int wide, ActBuf act, int64_t m4, cudaStream_t s);
int launch_binary(int op, const float *a, int64_t a_stride, const float *b, int64_t b_stride, int64_t b_ne0, int64_t b_rows,
                  float *y, int64_t y_stride, int64_t ne0, int64_t nrows, cudaStream_t s);
int launch_silu(const float *x, int64_t x_stride, const float *g, int64_t g_stride, float *y, int64_t y_stride, float *y_mul,
                int64_t y_mul_stride, int64_t ne0, int64_t nrows, int wide, cudaStream_t s);
void rope_table_host(const int32_t *pos, int64_t n_tok, int64_t ne0, const float *freq_factors, int n_dims, int n_ctx_orig,
                     float freq_base, float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow,
                     float *table);
int launch_rope(const float *x, int64_t x_nb1, int64_t x_nb2, float *y, int64_t y_nb1, int64_t y_nb2, const float *table,
                const int32_t *rows, int64_t n_rows, int64_t ne0, int64_t n_head, int64_t n_tok, int n_dims, int mode, cudaStream_t s);
unsigned long long scratch_generation();
int launch_set_rows_f16(const float *x, int64_t x_stride, const int64_t *idx, void *dst, int64_t dst_stride, int64_t dst_rows,
                        int64_t ne0, int64_t nrows, cudaStream_t s);
int launch_get_rows(int type, const void *table, int64_t ne0, int64_t table_rows, const int32_t *ids, int64_t n, float *out,
                    int64_t out_stride, cudaStream_t s);
int launch_argmax(const float *x, int64_t x_stride, int64_t ne0, int64_t nrows, int32_t *out, cudaStream_t s);

// scratch owned by the library (one growing allocation per device)
int scratch_get(size_t bytes, void **ptr);
int scratch_get_kx(size_t bytes, void **ptr);   // a second block, for the K-split exchange of the decode mat-mul
int scratch_get_lists(size_t bytes, void **ptr);   // a third, for attention's visible-position lists
int scratch_get_images(size_t bytes, void **ptr);  // a fourth, for the prompt mat-mul's f16 operand images (the activations sit in the first)
// graph_compute brackets a node list with (true) / (false): inside, attention reuses the lists of an unchanged mask
void flash_attn_graph_scope(bool enter);

// b200_mul_mat_static_scratch brackets its launches with this scope: inside it no route that needs a library
// scratch block is taken, and scratch_get* refuse instead of allocating (thread-local)
struct NoScratchScope {
    NoScratchScope();
    ~NoScratchScope();
};
bool no_scratch_mode();
// device allocations the library itself has made so far (scratch blocks); exported as b200_debug_alloc_count
unsigned long long library_alloc_count();
void gemv_stream_debug_wait(int spin_limit, int skip_unit);
// decode_persistent.cu: test hooks (see b200_debug_decode_step_*)
void decode_persistent_debug(int spin_limit, int skip_cta, int skip_barrier);
unsigned long long decode_persistent_launches();
int decode_persistent_times(unsigned long long *out, int n);
int gemm_fast_profile(unsigned long long *out, int n);            // gemm_tcgen05_fast.cu
void gemm_fast_debug_wait(int spin_limit, int mute_cta);          // gemm_tcgen05_fast.cu: test hook
int gemm_fast_reset_flags();                                      // gemm_tcgen05_fast.cu: the partial-tile flags of the current device, all down
int flash_attn_prefill_profile(unsigned long long *out, int n);   // flash_attn_prefill_tc.cu

// route the reference takes for (type, n, m), and the activation quantizer that route reads
int pick_route(int type, int64_t n, int64_t m);
int act_kind_for(int type, int route, int64_t m);

// ---- programmatic dependent launch ---------------------------------------------
// Kernels launched through launch_pdl() may start while the previous kernel in the stream is still
// running.  Each of them calls pdl_trigger() early (so that its own successor may start) and
// pdl_wait() before it reads anything a previous kernel wrote or writes anything a previous kernel
// reads; what they do before pdl_wait() (index set-up, streaming the weights in) overlaps the tail of
// the previous kernel.  B200_PDL=0 in the environment turns the attribute off.
bool pdl_enabled();
// 1 = tolerance-mode kernels where they exist, 0 = bit-exact reproduction of the CPU routes (b200_set_numerics)
int numerics_mode();
void set_numerics_mode(int mode);
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    return B200_STATUS_SUCCESS;
}
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

// ---- device helpers ----------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 16-byte streaming load: weights are read exactly once, keep them out of L1
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float e8m0_half_to_f32(uint32_t e) {
    // 2^(e-128): crates/ggml/src/quants.rs:682-691
    uint32_t bits = e < 2 ? (0x00200000u << e) : ((e - 1) << 23);
    return __uint_as_float(bits);
}
#endif

}  // namespace b200
