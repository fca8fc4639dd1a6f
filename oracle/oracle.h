// CPU oracle for the quantized mat-mul / flash-attention hot path.
//
// TEST INFRASTRUCTURE ONLY. This is a scalar restatement of the reference's
// CPU arithmetic (the Rust ggml crate), used by the tests as the checker and by
// the benchmark as the timed CPU baseline. Nothing in the shipped CUDA library
// links, loads or calls it.
//
// Every function names the reference file:line whose arithmetic it follows.
// All f32 arithmetic is written with explicit fmaf() where the reference fuses
// and is compiled with -ffp-contract=off so nothing else is fused.
#pragma once
#include <cstddef>
#include <cstdint>

#define QK_K 256
#define QK4_0 32
#define QK8_0 32
#define QK_MXFP4 32
#define K_SCALE_SIZE 12

// ggml type ids (GGUF wire ids): crates/ggml/src/types.rs:15-53
enum OrcType : int {
    ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q8_0 = 8, ORC_Q4_K = 12,
    ORC_Q6_K = 14, ORC_Q8_K = 15, ORC_MXFP4 = 39,
};

#pragma pack(push, 1)
// crates/ggml/src/blocks.rs:30-36
struct block_q4_0 { uint16_t d; uint8_t qs[QK4_0 / 2]; };
// crates/ggml/src/blocks.rs:47-53
struct block_mxfp4 { uint8_t e; uint8_t qs[QK_MXFP4 / 2]; };
// crates/ggml/src/blocks.rs:83-89
struct block_q8_0 { uint16_t d; int8_t qs[QK8_0]; };
// crates/ggml/src/blocks.rs:137-144
struct block_q4_K { uint16_t d; uint16_t dmin; uint8_t scales[K_SCALE_SIZE]; uint8_t qs[QK_K / 2]; };
// crates/ggml/src/blocks.rs:156-163
struct block_q6_K { uint8_t ql[QK_K / 2]; uint8_t qh[QK_K / 4]; int8_t scales[QK_K / 16]; uint16_t d; };
// crates/ggml/src/blocks.rs:165-172
struct block_q8_K { float d; int8_t qs[QK_K]; int16_t bsums[QK_K / 16]; };
#pragma pack(pop)

static_assert(sizeof(block_q4_0) == 18, "q4_0");
static_assert(sizeof(block_mxfp4) == 17, "mxfp4");
static_assert(sizeof(block_q8_0) == 34, "q8_0");
static_assert(sizeof(block_q4_K) == 144, "q4_K");
static_assert(sizeof(block_q6_K) == 210, "q6_K");
static_assert(sizeof(block_q8_K) == 292, "q8_K");

extern "C" {

// ---- scalar helpers -------------------------------------------------------
uint16_t orc_f32_to_f16(float x);
float orc_f16_to_f32(uint16_t h);
float orc_e8m0_to_f32_half(uint8_t e);
size_t orc_row_size(int type, int64_t k);   // bytes of one row of k elements
int orc_block_elems(int type);

// ---- weight quantizers / dequantizers ------------------------------------
// 0 on success, -1 for an unsupported type or a k that is not a block multiple
int orc_quantize_row(int type, const float *x, void *y, int64_t k);
int orc_dequantize_row(int type, const void *x, float *y, int64_t k);
int orc_quantize_rows(int type, const float *x, void *y, int64_t rows, int64_t k);

// ---- activation quantizers (A1..A4) --------------------------------------
void orc_quantize_row_q8_0(const float *x, void *y, int64_t k);            // A1
void orc_quantize_row_q8_K(const float *x, void *y, int64_t k);            // A2
void orc_quantize_mat_q8_K_4x8(const float *x, int64_t k, int64_t n_rows, void *out);  // A3
void orc_quantize_mat_q8_0_4x8(const float *x, int64_t k, int64_t n_rows, void *out);  // A4

// ---- 8x8 interleaved layouts (CPU_REPACK) --------------------------------
int orc_repack_8x8(int type, const void *src, int64_t nrows, int64_t k, void *dst);

// ---- row dots -------------------------------------------------------------
float orc_vec_dot(int type, int64_t k, const void *w_row, const void *act_row);

// ---- 8x8 kernels on the interleaved layouts (fixture replay) --------------
int orc_gemv_8x8(int type, int64_t k, float *s, const void *vx, const void *vy, int64_t nc);
int orc_gemm_8x8(int type, int64_t k, float *s, int64_t bs, const void *vx, const void *vy,
                 int64_t nr, int64_t nc);

// ---- graph-level ops ------------------------------------------------------
// Route selector for orc_mul_mat: 0 = what the reference picks for this
// (type, N, M); the others force one route so each can be pinned alone.
enum OrcRoute : int {
    ORC_ROUTE_AUTO = 0,
    ORC_ROUTE_ROWDOT = 1,   // vec_dot_row per (row, column)
    ORC_ROUTE_REPACK = 2,   // 8x8 gemm for 4-row groups + gemv tails
    ORC_ROUTE_TILED = 3,    // tiled K-quant kernel
};
// W: [N rows][K] quantized (plain ggml blocks), X: [M][K] f32, out: [M][N] f32
// (out[m*N + n], ggml dst layout ne0 = N).  Returns the route taken (>0) or -1.
int orc_mul_mat(int type, int64_t N, int64_t K, int64_t M, const void *W, const float *X,
                float *out, int route, int n_threads);

// MUL_MAT_ID. W: [n_expert][N][K]; B: [n_tok][ne11][K] f32; ids: [n_tok][n_ids]
// i32; out: [n_tok][n_ids][N].  Returns route or -1.
int orc_mul_mat_id(int type, int64_t N, int64_t K, int64_t n_expert, int64_t ne11, int64_t n_tok,
                   int64_t n_ids, const void *W, const float *B, const int32_t *ids, float *out,
                   int route, int n_threads);

// FLASH_ATTN_EXT.  q: [T][H][DK] f32 is NOT the layout: see oracle_flash_attn.cpp
// for the strides.  mode: 0 auto, 1 one_chunk, 2 split-KV (n_chunks), 3 tiled.
struct OrcFlashArgs {
    int64_t dk, dv, T, H, H_kv, n_kv;
    const float *q;       int64_t q_nb1, q_nb2;         // bytes: per token, per head
    const uint16_t *k;    int64_t k_nb1, k_nb2;         // bytes: per position, per kv head
    const uint16_t *v;    int64_t v_nb1, v_nb2;
    const uint16_t *mask; int64_t mask_nb1;             // f16 [T][n_kv] or null
    const float *sinks;                                 // [H] or null
    float scale, max_bias, logit_softcap;
    float *dst;                                         // [T][H][DV]
    int mode; int n_chunks; int n_threads;
};
int orc_flash_attn_ext(const OrcFlashArgs *a);

int orc_mul_mat_repacked(int type, int64_t N, int64_t K, int64_t M, const void *Wrep, const float *X,
                         float *out, int n_threads);
int orc_num_threads();
// Vector forms of the Q4_K 8x8 tile core and the Q6_K row dot (oracle_simd.cpp): the same exact integers, so every
// result stays bit-identical.  orc_set_simd caps the level (0 scalar, 1 AVX2, 2 AVX-512 VNNI; default 2);
// orc_simd_level is what runs on this host under the cap.
void orc_set_simd(int max_level);
int orc_simd_level(void);
int orc_pick_route(int type, int64_t N, int64_t M);   // the route orc_mul_mat takes with ORC_ROUTE_AUTO

}  // extern "C"
