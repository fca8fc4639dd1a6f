/* ggml_b200.h — C ABI of libggml-b200.so, a CUDA (sm_100a) implementation of
 * the ggml quantized mat-mul / flash-attention hot path.
 *
 * Two faces:
 *   1. op-level entry points (this file): plain pointers and sizes, what an
 *      FFI crate binds when it wants one op at a time;
 *   2. the ggml backend plug-in vtables (ggml_b200_backend.h): what the ggml
 *      crate's registry loads with dlopen and drives through graph_compute.
 *
 * Every entry point returns a ggml status code and never aborts:
 * crates/ggml/src/backend.rs:54-62 (GgmlStatus).
 */
#ifndef GGML_B200_H
#define GGML_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* enum ggml_status — crates/ggml/src/backend.rs:54-62, sysffi.rs:360-364 */
enum b200_status {
    B200_STATUS_SUCCESS = 0,
    B200_STATUS_ALLOC_FAILED = 1,
    B200_STATUS_OUT_OF_MEMORY = 2,
    B200_STATUS_BACKEND_ERROR = 3,
    B200_STATUS_ABORTED = 4,
    /* argument errors are reported as BACKEND_ERROR + b200_last_error() text */
};

/* enum ggml_type (GGUF wire ids) — crates/ggml/src/types.rs:15-53 */
enum b200_type {
    B200_TYPE_F32 = 0,
    B200_TYPE_F16 = 1,
    B200_TYPE_Q4_0 = 2,
    B200_TYPE_Q8_0 = 8,
    B200_TYPE_Q4_K = 12,
    B200_TYPE_Q6_K = 14,
    B200_TYPE_Q8_K = 15,
    B200_TYPE_I32 = 26,
    B200_TYPE_I64 = 27,
    B200_TYPE_MXFP4 = 39,
};

/* Activation quantizers of the CPU path (which Q8 blocks an op builds):
 *   A1 quantize_row_q8_0       crates/ggml/src/quants.rs:331-362
 *   A2 quantize_row_q8_K       crates/ggml/src/quants.rs:615-654
 *   A3 quantize_mat_q8_K_4x8   crates/ggml/src/repack.rs:1561-1606 (values) */
enum b200_act_quant {
    B200_ACT_Q8_0 = 1, B200_ACT_Q8_K = 2, B200_ACT_Q8_K_4X8 = 3,
    /* what the Q4_K 8x8 route builds: A3 for the complete groups of 4 rows, A2 for the m % 4 tail
     * (crates/ggml/src/compute.rs:5322-5400) */
    B200_ACT_Q8_K_MIXED = 4,
};

/* Which CPU route's arithmetic a mat-mul reproduces (crates/ggml/src/compute.rs:1420-1841).
 * AUTO picks what the reference picks for (type, N, M). */
enum b200_route { B200_ROUTE_AUTO = 0, B200_ROUTE_ROWDOT = 1, B200_ROUTE_REPACK = 2, B200_ROUTE_TILED = 3 };

/* ---- library / device ---------------------------------------------------- */
const char *b200_last_error(void);             /* thread-local text of the last failure */
int b200_device_count(void);                   /* 0 when no CUDA device is usable */
int b200_set_device(int device);
int b200_device_info(int device, char *name, size_t name_len, size_t *free_bytes, size_t *total_bytes,
                     int *sm_count, int *cc_major, int *cc_minor);
int b200_synchronize(void *stream);
/* Numerics policy.  B200_NUMERICS_EXACT: every kernel reproduces, bit for bit, the arithmetic of the CPU route the
 * reference takes for the op (activation blocks, integer block dots, the f32 chains in their order, the f16
 * attention accumulator).  B200_NUMERICS_FAST (the start value unless the environment says B200_NUMERICS=exact):
 * ops for which a tolerance-mode kernel exists use it, within the tolerances asked of this path (1e-5 of
 * sum |w x| per mat-mul output, 1e-3 for F16-KV attention); the others stay exact.  Process-wide; takes effect at the
 * next call.  (The reference's own routes for one op differ by about 1e-6: crates/llama/tests/gpt_oss_e2e.rs:63-64.) */
enum b200_numerics { B200_NUMERICS_EXACT = 0, B200_NUMERICS_FAST = 1 };
void b200_set_numerics(int mode);
int b200_get_numerics(void);
/* Kernels that wait on barriers bound every wait; a wait that ran out records a non-zero code on the
 * device instead of hanging it.  Reads and clears that code for the current device (0 = none).
 * (Failure reporting of the kind ggml_backend_i.synchronize surfaces: crates/ggml/src/backend.rs:761-765.) */
int b200_kernel_error(int *code);
/* Test hooks (no counterpart in the reference).  b200_debug_alloc_count: device allocations the library has made
 * for its own scratch blocks so far in this process.  b200_debug_stream_wait: while spin_limit > 0, one-row Q4_K
 * mat-muls of few row tiles take the bulk-copy streaming kernel (selectable otherwise with B200_GEMV_STREAM=1),
 * its waits poll at most spin_limit times, and its producer leaves ring unit skip_unit unfilled (-1 = none), so
 * that a test can watch a bounded wait run out: the kernel returns, its output rows stay unwritten and
 * b200_kernel_error reports code 1 (producer) or 2 (consumer).  spin_limit 0 disarms the hook.
 * b200_debug_decode_step_launches: how many one-token steps the backend has run as its single persistent kernel so far
 * in this process (a test that compares it with the node-by-node path first checks that it was taken at all).
 * b200_debug_decode_step_wait: while spin_limit > 0 every wait of that kernel polls at most spin_limit times and CTA
 * skip_cta never arrives at its grid barrier number skip_barrier (-1 = none): the others' wait runs out, the kernel
 * returns with its outputs unfinished and b200_kernel_error reports code 5.  spin_limit 0 disarms the hook. */
unsigned long long b200_debug_alloc_count(void);
void b200_debug_stream_wait(int spin_limit, int skip_unit);
unsigned long long b200_debug_decode_step_launches(void);
/* profiling aid: the device clock (ns) at which CTA 0 of the last persistent step started and passed each of its grid
 * barriers; call after synchronizing; returns how many stamps were copied (0 where there is nothing to read) */
int b200_debug_decode_step_times(unsigned long long *out, int n);
/* profiling aid: with B200_FA_PREFILL_PROFILE=1 in the environment the tcgen05 prompt-attention kernel sums, for one thread
 * of each role of its first CTA, the SM clocks spent at each barrier and at work (24 counters); this reads them back */
int b200_debug_fa_prefill_profile(unsigned long long *out, int n);
/* profiling aid: with B200_GEMM_FAST_PROFILE=1 the fast-numerics Q4_K prompt mat-mul sums, for one thread of each role of its
 * first CTA, the SM clocks spent at each barrier and at work (10 counters); this reads them back and clears them */
int b200_debug_gemm_fast_profile(unsigned long long *out, int n);
/* test hook: the fast-numerics prompt mat-mul cuts its work into one run per CTA, and a tile cut between CTAs is finished by
 * the CTA holding its first part, which waits (bounded) for the others' partial tiles.  While spin_limit > 0 that wait polls
 * at most spin_limit times and CTA mute_cta never announces its partial tile: the wait runs out, the kernel returns with that
 * tile unwritten and b200_kernel_error reports code 4.  spin_limit 0 disarms the hook. */
void b200_debug_gemm_fast_wait(int spin_limit, int mute_cta);
/* test hook: the persistent few-rows Q4_K mat-mul (8 to 31 activation rows) hands ring slots from a producer warp to multiply
 * warps to chain warps through barriers.  While spin_limit > 0 its waits poll at most spin_limit times and the producer of the
 * launch's first CTA leaves its unit skip_unit unfilled (-1 = none): a wait runs out, the kernel returns with that CTA's rows
 * unwritten and b200_kernel_error reports code 4.  spin_limit 0 disarms the hook. */
void b200_debug_rows_ring_wait(int spin_limit, int skip_unit);
void b200_debug_decode_step_wait(int spin_limit, int skip_cta, int skip_barrier);
/* Which kernel a Q4_K prompt mat-mul (8x8 gemm route, n weight rows, m >= 32 activation rows) takes on a GPU with
 * sm_count SMs: 0 = integer tcgen05 kernel, 3 / 4 = the two-pass f16-image kernels with 64 / 128 activation rows
 * per CTA.  Pure host arithmetic (CTA waves times measured time per wave, plus the expansion); no CUDA call.
 * (The reference's own choice among its gemm kernels by shape: crates/ggml/src/compute.rs:1420-1841.) */
int b200_prompt_kernel_choice(int64_t n, int64_t m, int sm_count);

/* ---- device memory (cudaMalloc-backed; buffers of the backend use the same) */
int b200_malloc(void **dev_ptr, size_t bytes);
int b200_free(void *dev_ptr);
int b200_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes, void *stream);
int b200_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes, void *stream);
int b200_memset(void *dev_dst, int value, size_t bytes, void *stream);
int b200_host_alloc_pinned(void **host_ptr, size_t bytes);
int b200_host_free_pinned(void *host_ptr);

/* ---- weights: device tile layout ------------------------------------------
 * Quantized tensors live on the device in a 32-row interleaved tile layout
 * (same bytes, re-ordered so that a warp reads 512 contiguous bytes per load).
 * This replaces the CPU path's load-time CPU_REPACK interleave
 * (crates/ggml/src/repack.rs:165,1435,3260; cache crates/ggml/src/compute.rs:698-775).
 * n_rows = ne01 * ne02 * ne03 (experts are stacked rows), k = ne00. */
size_t b200_weight_nbytes(int type, int64_t n_rows, int64_t k);   /* 0 = unsupported shape */
/* host ggml blocks (row-major, ggml row size) -> device tile layout */
int b200_weight_upload(int type, int64_t n_rows, int64_t k, const void *host_blocks, void *dev_tiles,
                       void *stream);
/* device tile layout -> host ggml blocks (round trip of the above) */
int b200_weight_download(int type, int64_t n_rows, int64_t k, const void *dev_tiles, void *host_blocks,
                         void *stream);
/* dequantize_row(ty, ..) of every row: crates/ggml/src/quants.rs:1098 */
int b200_dequantize(int type, int64_t n_rows, int64_t k, const void *dev_tiles, float *dev_out, void *stream);

/* ---- activations ------------------------------------------------------------
 * Runs the device quantizer on dev_x [m][k] f32 and returns the blocks in the
 * CPU path's own byte layout (block_q8_0 / block_q8_K rows; block_q8_Kx4 tiles
 * for A3, m % 4 == 0), for bit-exact comparison. */
int b200_quantize_activations(int kind, int64_t m, int64_t k, const float *dev_x, void *host_blocks,
                              void *stream);

/* Device-side form of the same quantizers for callers that own the scratch:
 * dev_act must hold b200_act_scratch_nbytes(m, k) bytes (256-byte aligned). One
 * quantized activation can feed several mat-muls (wq/wk/wv read the same row). */
size_t b200_act_scratch_nbytes(int64_t m, int64_t k);
int b200_quantize_activations_device(int kind, int64_t m, int64_t k, const float *dev_x, int64_t ldx,
                                     void *dev_act, void *stream);

/* ---- events (timing on the launching stream; ggml's event_record / event_synchronize,
 * crates/ggml/src/backend.rs:652-669) */
int b200_event_create(void **event);
int b200_event_destroy(void *event);
int b200_event_record(void *event, void *stream);
int b200_event_synchronize(void *event);
int b200_event_elapsed_ms(void *start, void *stop, float *ms);

/* ---- MUL_MAT — crates/ggml/src/compute.rs:1420 (forward_mul_mat), ops.rs:1329
 * dst[m][n] = sum_k W[n][k] * X[m][k]; W in device tile layout, X/dst f32 on
 * the device (row strides in elements).  route: enum b200_route. */
int b200_mul_mat(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const float *dev_x,
                 int64_t ldx, float *dev_dst, int64_t lddst, int route, void *stream);
/* the mat-mul proper on activations already quantized by
 * b200_quantize_activations_device (act_kind must be the kind the route reads) */
int b200_mul_mat_q8(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const void *dev_act,
                    int act_kind, float *dev_dst, int64_t lddst, int route, void *stream);
/* b200_mul_mat_q8 for one activation row that also writes dev_sum[i] = dst[i] + dev_addend[i] (one rounded
 * f32 add per element): the residual ADD that follows attn_output and ffn_down in a decoder layer
 * (crates/llama/src/graph_arch.rs:209,226; crates/ggml/src/compute.rs:1174) without a second kernel. */
int b200_mul_mat_q8_add(int type, int64_t n, int64_t k, const void *dev_w, const void *dev_act, int act_kind, float *dev_dst,
                        const float *dev_addend, float *dev_sum, int route, void *stream);
/* The same for the 8 to 31 activation rows of a batched decode step (a multiple of 4 for Q4_K): every row c also gets
 * dev_sum[c * ld_sum + i] = dst[c * lddst + i] + dev_addend[c * ld_addend + i].  Only the shapes the few-rows kernels take:
 * b200_mul_mat_q8_rows_add_fusable says (1 / 0) whether (type, n weight rows, m activation rows) is one; the call refuses the others. */
int b200_mul_mat_q8_rows_add_fusable(int type, int64_t n, int64_t m);
int b200_mul_mat_q8_rows_add(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const void *dev_act, int act_kind, float *dev_dst,
                             int64_t lddst, const float *dev_addend, int64_t ld_addend, float *dev_sum, int64_t ld_sum, void *stream);
/* Measurement helper (no counterpart in the reference): `reps` launches of b200_mul_mat_q8 over n_w rotating copies
 * of the weights (so that they come from HBM, not L2), captured into one CUDA graph and replayed, timed with events
 * on the launching stream.  This is what the kernel costs inside a decode step, where a replayed graph issues the
 * launches back to back; a host loop over b200_mul_mat_q8 measures the host's launch rate for small matrices. */
int b200_bench_mul_mat_q8(int type, int64_t n, int64_t k, int64_t m, const void *const *dev_w, int n_w, const void *dev_act,
                          int act_kind, float *dev_dst, int reps, float *us_per_launch);
/* b200_mul_mat_q8 for one activation row against up to three Q4_K matrices of the same k in one launch
 * (dev_dst[i][n[i]] = W_i x): the k / v / q mat-muls of an attention block and the gate / up mat-muls of an
 * FFN read the same normed row (crates/llama/src/graph_arch.rs:171-190,1137-1151), and at one token each of
 * them is a few microseconds of launch latency.  Every n[i] must take the 8x8 gemv route (a multiple of 8). */
int b200_mul_mat_q8_multi(int type, int64_t k, int count, const int64_t *n, const void *const *dev_w, const void *dev_act,
                          int act_kind, float *const *dev_dst, void *stream);
/* The same for m activation rows (prompt batches): count (1 .. 3) matrices of one type and row length against the same
 * quantized activations, dev_dst[i] [m][lddst[i]].  All matrices must take the same CPU route for m rows (the route b200_mul_mat_q8 picks under B200_ROUTE_AUTO).
 * In the exact numerics mode it gives exactly what count calls of b200_mul_mat_q8 give; where the fast-numerics prompt
 * kernel applies the matrices share one launch and one expansion of the activations, and the outputs agree with separate
 * calls within that mode's tolerance (the kernel's CTAs cut the tiles' f32 sums in other places) (the q / k / v and gate / up projections of a layer,
 * crates/llama/src/graph_arch.rs:171-190,1137-1151). */
int b200_mul_mat_q8_rows_multi(int type, int64_t k, int64_t m, int count, const int64_t *n, const void *const *dev_w, const void *dev_act, int act_kind,
                               float *const *dev_dst, const int64_t *lddst, void *stream);
/* One-row Q4_K mat-mul(s) with the f32 op in front of them and the Q8_K quantization of its result run inside the
 * mat-mul kernel (at one token each of those ops is a launch of a few microseconds for a few KB of work):
 *   B200_ACT_PRO_PLAIN  act = q8_K(x)                          — a mat-mul whose activations are not quantized yet
 *   B200_ACT_PRO_NORM   y = x * rms_scale(x, eps); y_mul = y * w; act = q8_K(y_mul)
 *                       — RMS_NORM + MUL in front of q/k/v and gate/up (crates/llama/src/graph_arch.rs:1119-1122)
 *   B200_ACT_PRO_SILU   y = silu(x); y_mul = y * w; act = q8_K(y_mul)
 *                       — SILU + MUL in front of ffn_down (crates/llama/src/graph_arch.rs:1137-1151); wide as in b200_silu
 * Element for element the arithmetic is that of b200_rms_norm / b200_silu, quantize_row_q8_K and b200_mul_mat_q8
 * (bit-identical results); y (may be null) and y_mul are written as the separate ops would write them, and
 * dev_act_out (may be null; b200_act_scratch_nbytes(1, k) bytes) receives the quantized row for later mat-muls.
 * Up to three matrices of the same k share the launch (dev_dst[i][n[i]]); with one matrix, dev_sum[n] (if given)
 * receives dst + dev_addend, the residual ADD that follows attn_output and ffn_down. */
enum { B200_ACT_PRO_PLAIN = 1, B200_ACT_PRO_NORM = 2, B200_ACT_PRO_SILU = 3 };
struct b200_act_prologue {
    int mode;
    const float *x;
    const float *w;
    float eps;
    int wide;
    float *y;
    float *y_mul;
    void *dev_act_out;
};
int b200_mul_mat_row_fused(int type, int64_t k, int count, const int64_t *n, const void *const *dev_w, float *const *dev_dst,
                           const struct b200_act_prologue *pro, const float *dev_addend, float *dev_sum, void *stream);
/* same op with host activations / results: copies X in, runs, copies dst out */
int b200_mul_mat_host(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const float *host_x,
                      float *host_dst, int route, void *stream);

/* b200_mul_mat for callers that must not allocate.  It has no counterpart in the
 * reference (whose CPU path takes its work buffer from the graph planner).
 * b200_mul_mat keeps the quantized activations in a block it gets from
 * cudaMalloc and may re-allocate; hosts that fixed their device-memory budget
 * up front, that route every allocation through their own memory manager, or
 * that call from a point where the allocator is out of reach use this form
 * instead: its scratch is a fixed 256 KiB array inside the loaded module
 * (b200_static_scratch_nbytes), one copy per device for the life of the
 * process, and the call performs no allocation of any kind: the kernels' error
 * word and counters are module variables as well, and where b200_mul_mat would
 * pick a kernel that needs a further scratch block (the two-pass prompt kernels)
 * this entry point runs the one-pass kernel that gives the same bits.
 *  - m x k activations whose quantized form exceeds the array are refused with
 *    B200_STATUS_BACKEND_ERROR and a message; nothing is launched.
 *  - The first call on a device resolves the array's device address (that
 *    device must be current); issue it before beginning any stream capture.
 *  - Every call on a device shares the array, which keeps the previous call's
 *    contents (none of it has to be zero on entry).  Calls in one stream are
 *    ordered; calls whose kernels may overlap on the GPU race on the array. */
size_t b200_static_scratch_nbytes(void);
int b200_mul_mat_static_scratch(int type, int64_t n, int64_t k, int64_t m, const void *dev_w,
                                const float *dev_x, int64_t ldx, float *dev_dst, int64_t lddst, int route,
                                void *stream);

/* ---- MUL_MAT_ID — crates/ggml/src/compute.rs:1917 (forward_mul_mat_id), ops.rs:1421
 * as: [n_expert][n][k] tiles (stacked rows); b: [n_tok][ne11][k] f32;
 * ids: [n_tok][n_ids] i32; dst: [n_tok][n_ids][n] f32.  All device pointers. */
int b200_mul_mat_id(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok,
                    int64_t n_ids, const void *dev_as, const float *dev_b, const int32_t *dev_ids,
                    float *dev_dst, int route, void *stream);

/* ---- FLASH_ATTN_EXT — crates/ggml/src/compute.rs:4563, flash_attn.rs:907,920, ops.rs:2430
 * q f32 [T][H][DK] by byte strides, k/v f16 by byte strides (KV-cache views,
 * crates/llama/src/kv_cache.rs:2528-2579), mask f16 [T][n_kv] or NULL,
 * dst f32 [T][H][DV] contiguous.
 * The CPU result for one query row over >= 512 positions depends on the CPU
 * thread count (split-KV, flash_attn.rs:841-859): n_chunks names the thread
 * count to reproduce (0 = 8, the count the reference's benchmark scripts use).
 * mode 0 follows the library's numerics policy (b200_set_numerics); mode 2 reproduces the CPU arithmetic
 * (f16 accumulator order and all); mode 1 is the fast path with f32 accumulation (more accurate than the
 * CPU, not bit-comparable to it; shapes it does not cover — sinks, ALiBi, softcap, dk != dv — take the
 * exact kernels). */
struct b200_flash_attn_args {
    int64_t dk, dv, n_tok, n_head, n_head_kv, n_kv;
    const float *q;      int64_t q_nb1, q_nb2;     /* bytes per token, per head */
    const void *k;       int64_t k_nb1, k_nb2;     /* bytes per position, per kv head */
    const void *v;       int64_t v_nb1, v_nb2;
    const void *mask;    int64_t mask_nb1;         /* bytes per token row */
    const float *sinks;                            /* [n_head] or NULL */
    float scale, max_bias, logit_softcap;
    float *dst;
    int32_t n_chunks;
    int32_t mode;
};
int b200_flash_attn_ext(const struct b200_flash_attn_args *args, void *stream);

/* ---- the f32 ops between the mat-muls of a decoder layer -------------------------------------------
 * Each replaces one arm of the CPU engine's dispatch (crates/ggml/src/compute.rs:1026-1110) and performs
 * the same rounded operations per element.  Pointers are device pointers; row strides count elements
 * unless the name says nb (bytes).  Rows hold ne0 dense elements. */

/* RMS_NORM, crates/ggml/src/compute.rs:2634-2683.  y may be null when only the weighted result is wanted.
 * With weight != null also writes y_weighted = (x * scale) * weight[i], the MUL that follows the norm in
 * every decoder (crates/llama/src/graph_arch.rs:1119-1122). */
int b200_rms_norm(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *weight, float *y_weighted,
                  int64_t y_weighted_stride, int64_t ne0, int64_t nrows, float eps, void *stream);

/* b200_rms_norm / b200_silu (below) that also leave the Q8_K quantization of their last result (the
 * weighted norm, the gated product) in dev_act for the mat-muls that read it — the CPU engine quantizes
 * that tensor at the head of each MUL_MAT (crates/ggml/src/compute.rs:1466-1500); here the producer does it
 * once.  dev_act: b200_act_scratch_nbytes(nrows, ne0) bytes, 256-byte aligned; act_kind: one of the Q8_K
 * kinds of enum b200_act_quant (what b200_mul_mat_q8 will be given); ne0 a multiple of 256. */
int b200_rms_norm_q8(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *weight, float *y_weighted,
                     int64_t y_weighted_stride, int64_t ne0, int64_t nrows, float eps, void *dev_act, int act_kind, void *stream);
int b200_silu_q8(const float *x, int64_t x_stride, const float *gate, int64_t gate_stride, float *y, int64_t y_stride, float *y_gated,
                 int64_t y_gated_stride, int64_t ne0, int64_t nrows, int wide, void *dev_act, int act_kind, void *stream);

/* ADD (op 0) / MUL (op 1) of F32 tensors with ggml's row broadcast, crates/ggml/src/compute.rs:1174-1330:
 * y[r][i] = a[r][i] op b[r % b_rows][i % b_ne0]. */
int b200_binary(int op, const float *a, int64_t a_stride, const float *b, int64_t b_stride, int64_t b_ne0, int64_t b_rows, float *y,
                int64_t y_stride, int64_t ne0, int64_t nrows, void *stream);

/* UNARY(SILU), crates/ggml/src/compute.rs:3109-3135 -> crates/ggml/src/simd_x86.rs:1012-1054.  wide != 0
 * reproduces a host with AVX512F+DQ (16-lane chunks through the polynomial exp, the row tail through libm
 * expf), wide == 0 a host without (libm throughout); b200_host_silu_is_wide() reports this host.  With
 * gate != null also writes y_gated = silu(x) * gate, the MUL that follows in the FFN
 * (crates/llama/src/graph_arch.rs:1150-1151). */
int b200_silu(const float *x, int64_t x_stride, const float *gate, int64_t gate_stride, float *y, int64_t y_stride, float *y_gated,
              int64_t y_gated_stride, int64_t ne0, int64_t nrows, int wide, void *stream);
int b200_host_silu_is_wide(void);

/* ROPE, crates/ggml/src/compute.rs:3679-3800, modes NORMAL (0) and NEOX (2), F32.
 * b200_rope_table fills a HOST table [n_tok][ne0] of (cos, sin) pairs from HOST positions with the host
 * libm, as rope_cache_init (:3539-3566) does; freq_factors is a host array of ne0/2 floats or null.
 * b200_rope rotates x [ne0, n_head, n_tok] (byte strides nb1 per head, nb2 per token) into y with a copy
 * of that table in device memory: token t uses table row t, or, when table_rows (device, I32 [n_tok]) is
 * given, row table_rows[t] of a table of table_n_rows rows — a table built once for positions
 * 0 .. table_n_rows-1 then serves every step with the position tensor as the index.  An index outside
 * the table skips the token and b200_kernel_error() reports code 3. */
int b200_rope_table(const int32_t *pos, int64_t n_tok, int64_t ne0, const float *freq_factors, int n_dims, int n_ctx_orig,
                    float freq_base, float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow,
                    float *table);
int b200_rope(const float *x, int64_t x_nb1, int64_t x_nb2, float *y, int64_t y_nb1, int64_t y_nb2, const float *table,
              const int32_t *table_rows, int64_t table_n_rows, int64_t ne0, int64_t n_head, int64_t n_tok, int n_dims, int mode,
              void *stream);

/* SET_ROWS of F32 rows into an F16 destination with I64 indices (the KV-cache write),
 * crates/ggml/src/compute.rs:4265-4338.  A row whose index is outside [0, dst_rows) is skipped and
 * b200_kernel_error() reports code 2 afterwards (the CPU engine asserts). */
int b200_set_rows_f16(const float *x, int64_t x_stride, const int64_t *idx, void *dst, int64_t dst_stride, int64_t dst_rows,
                      int64_t ne0, int64_t nrows, void *stream);

/* GET_ROWS to F32, crates/ggml/src/compute.rs:3842-3895.  table: F32 or F16 dense rows, or a quantized
 * tensor in the tile layout of b200_weight_upload.  An id outside [0, table_rows) is skipped and
 * b200_kernel_error() reports code 1 afterwards (the CPU engine asserts). */
int b200_get_rows(int type, const void *table, int64_t ne0, int64_t table_rows, const int32_t *ids, int64_t n, float *y,
                  int64_t y_stride, void *stream);

/* ARGMAX per row, the last index among equal maxima, crates/ggml/src/compute.rs:4208-4228. */
int b200_argmax(const float *x, int64_t x_stride, int64_t ne0, int64_t nrows, int32_t *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GGML_B200_H */
