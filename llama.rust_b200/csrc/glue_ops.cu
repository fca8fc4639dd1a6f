// The f32 ops between the quantized mat-muls of a decoder layer: RMS_NORM, ADD / MUL, SILU, ROPE,
// SET_ROWS into an F16 cache, GET_ROWS, ARGMAX.  Each kernel performs the same rounded operations per
// element as the reference's CPU engine, so a layer's activations reach the next mat-mul's quantizer
// with the bits the CPU path would have given them.  All of them are bound by launch latency at one
// token and by HBM at a prompt batch; rows are read and written with coalesced 16-byte accesses.
#include <cmath>
#include <cstring>

#include "common.cuh"
#include "act_quant.cuh"
#include "fa_math.cuh"

namespace b200 {

// ---- RMS_NORM (+ optional weight MUL) -----------------------------------------------------------
// crates/ggml/src/compute.rs:2634-2683: sum of the f32 squares in f64, mean narrowed to f32,
// scale = 1 / sqrt(mean + eps), y = x * scale.  The f64 partial sums are combined in a tree instead of
// element order; f64 keeps 29 more bits than the f32 mean needs, so the narrowed mean is the same.
// With w != nullptr the kernel also emits (x * scale) * w[i] (crates/llama/src/graph_arch.rs:1119-1122),
// each product rounded on its own.  One CTA per row.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float *__restrict__ x, int64_t x_stride, float *y, int64_t y_stride, const float *__restrict__ w,
                float *y_mul, int64_t y_mul_stride, int ne0, float eps) {
    pdl_trigger();
    pdl_wait();
    const float *xr = x + (int64_t)blockIdx.x * x_stride;
    double sum = 0.0;
    for (int i = threadIdx.x; i < ne0; i += 256) {
        const float v = xr[i];
        sum += (double)__fmul_rn(v, v);
    }
    __shared__ double part[8];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) total += part[i];
    const float mean = __double2float_rn(total / (double)ne0);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    for (int i = threadIdx.x; i < ne0; i += 256) {
        const float n = __fmul_rn(xr[i], scale);
        if (y) y[(int64_t)blockIdx.x * y_stride + i] = n;
        if (w) y_mul[(int64_t)blockIdx.x * y_mul_stride + i] = __fmul_rn(n, w[i]);
    }
}

int launch_rms_norm(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *w, float *y_mul,
                    int64_t y_mul_stride, int64_t ne0, int64_t nrows, float eps, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30), "rms_norm: bad row length %lld", (long long)ne0);
    B200_REQUIRE(nrows < 0x7fffffffLL, "rms_norm: too many rows");
    if (nrows == 0) return B200_STATUS_SUCCESS;
    return launch_pdl(rms_norm_kernel, dim3((unsigned)nrows), dim3(256), 0, s, x, x_stride, y, y_stride, w, y_mul, y_mul_stride,
                      (int)ne0, eps);
}

// Few rows (single-token and small-batch steps, where latency counts and there are not enough rows to fill the GPU
// with one CTA each): the same, followed by the Q8_K quantization of the result for the mat-muls that read it: grid
// (ne0 / 256, rows), every CTA recomputes the row's sum (the row is a few KB and sits in L2) in the same
// order, then owns one 256-element block: norm, weighted norm, and that block's quants, scale and
// 16-element sums (act_quant.cuh).  Rows below m4 take the 4x8 value rule, the others the plain one.
__global__ void __launch_bounds__(256)
rms_norm_q8_few_kernel(const float *__restrict__ x, int64_t x_stride, float *y, int64_t y_stride, const float *__restrict__ w,
                   float *y_mul, int64_t y_mul_stride, int ne0, float eps, ActBuf act, int64_t m4) {
    pdl_trigger();
    pdl_wait();
    const int64_t row = blockIdx.y;
    const float *xr = x + row * x_stride;
    double sum = 0.0;
    for (int i = threadIdx.x; i < ne0; i += 256) {
        const float v = xr[i];
        sum += (double)__fmul_rn(v, v);
    }
    __shared__ double part[8];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) total += part[i];
    const float mean = __double2float_rn(total / (double)ne0);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    const int i = blockIdx.x * 256 + threadIdx.x;
    const float n = __fmul_rn(xr[i], scale);
    if (y) y[row * y_stride + i] = n;
    float v = n;
    if (w) {
        v = __fmul_rn(n, w[i]);
        y_mul[row * y_mul_stride + i] = v;
    }
    if (row < m4) q8_K_block_store<true>(v, act, row, blockIdx.x);
    else q8_K_block_store<false>(v, act, row, blockIdx.x);
}

// eight consecutive floats, as two 16-byte accesses when every operand of the launch allows it (vec), else one by one
__device__ __forceinline__ void load8(const float *p, bool vec, float (&v)[8]) {
    if (vec) {
        const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = p[j];
    }
}
__device__ __forceinline__ void store8(float *p, bool vec, const float (&v)[8]) {
    if (vec) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) p[j] = v[j];
    }
}

// Many rows (prompt batches): the same with one CTA per row:
// the row's sum in the same order as above, then warp w takes the 256-element blocks w, w + 8, ..: lane l
// holds elements 8 l .. 8 l + 7, writes norm and weighted norm with 16-byte stores and the block's quants,
// scale and 16-element sums (act_quant.cuh).  Rows below m4 take the 4x8 value rule, the others the plain one.
__global__ void __launch_bounds__(256)
rms_norm_q8_kernel(const float *__restrict__ x, int64_t x_stride, float *y, int64_t y_stride, const float *__restrict__ w,
                   float *y_mul, int64_t y_mul_stride, int ne0, float eps, ActBuf act, int64_t m4, bool vec) {
    pdl_trigger();
    pdl_wait();
    const int64_t row = blockIdx.x;
    const float *xr = x + row * x_stride;
    double sum = 0.0;
    for (int i = threadIdx.x; i < ne0; i += 256) {
        const float v = xr[i];
        sum += (double)__fmul_rn(v, v);
    }
    __shared__ double part[8];
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) total += part[i];
    const float mean = __double2float_rn(total / (double)ne0);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int blk = warp; blk < ne0 / 256; blk += 8) {
        const int i = blk * 256 + 8 * lane;
        float v[8];
        load8(xr + i, vec, v);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = __fmul_rn(v[j], scale);
        if (y) store8(y + row * y_stride + i, vec, v);
        if (w) {
            float ws[8];
            load8(w + i, vec, ws);
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = __fmul_rn(v[j], ws[j]);
            store8(y_mul + row * y_mul_stride + i, vec, v);
        }
        if (row < m4) q8_K_block_store_warp<true>(v, act, row, blk);
        else q8_K_block_store_warp<false>(v, act, row, blk);
    }
}

// up to this many rows the one-CTA-per-block kernels are used (measured: a single-token step loses 4 % with the row kernels)
constexpr int64_t FEW_ROWS = 32;
static bool aligned16(const void *p, int64_t stride_elems) { return ((uintptr_t)p & 15) == 0 && stride_elems % 4 == 0; }

int launch_rms_norm_q8(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *w, float *y_mul,
                       int64_t y_mul_stride, int64_t ne0, int64_t nrows, float eps, ActBuf act, int64_t m4, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 % 256 == 0 && ne0 < (1 << 30), "rms_norm + q8_K: row length %lld is not a multiple of 256", (long long)ne0);
    B200_REQUIRE(nrows < 0x7fffffffLL, "rms_norm + q8_K: too many rows");
    const bool vec = aligned16(x, x_stride) && (!y || aligned16(y, y_stride)) && (!w || (aligned16(w, 4) && aligned16(y_mul, y_mul_stride)));
    if (nrows == 0) return B200_STATUS_SUCCESS;
    if (nrows <= FEW_ROWS)
        return launch_pdl(rms_norm_q8_few_kernel, dim3((unsigned)(ne0 / 256), (unsigned)nrows), dim3(256), 0, s, x, x_stride, y, y_stride, w,
                          y_mul, y_mul_stride, (int)ne0, eps, act, m4);
    return launch_pdl(rms_norm_q8_kernel, dim3((unsigned)nrows), dim3(256), 0, s, x, x_stride, y, y_stride, w, y_mul, y_mul_stride,
                      (int)ne0, eps, act, m4, vec);
}

// ---- ADD / MUL -------------------------------------------------------------------------------------
// crates/ggml/src/compute.rs:1174-1330, F32 operands: y[r][i] = a[r][i] op b[r % b_rows][i % b_ne0].
template <int OP>
__global__ void __launch_bounds__(256)
binary_kernel(const float *__restrict__ a, int64_t a_stride, const float *__restrict__ b, int64_t b_stride, int b_ne0,
              int64_t b_rows, float *y, int64_t y_stride, int ne0, int64_t total) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / ne0;
    const int c = (int)(i - r * ne0);
    const float av = a[r * a_stride + c];
    const float bv = b[(r % b_rows) * b_stride + (b_ne0 == ne0 ? c : c % b_ne0)];
    y[r * y_stride + c] = OP == 0 ? __fadd_rn(av, bv) : __fmul_rn(av, bv);
}

// four elements per thread with 16-byte accesses: rows of a multiple of 4 floats, 16-byte aligned, b not broadcast along a row
template <int OP>
__global__ void __launch_bounds__(256)
binary_vec_kernel(const float *__restrict__ a, int64_t a_stride, const float *__restrict__ b, int64_t b_stride, int64_t b_rows, float *y,
                  int64_t y_stride, int ne0_4, int64_t total4) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total4) return;
    const int64_t r = i / ne0_4;
    const int c = 4 * (int)(i - r * ne0_4);
    const float4 av = *reinterpret_cast<const float4 *>(a + r * a_stride + c), bv = *reinterpret_cast<const float4 *>(b + (r % b_rows) * b_stride + c);
    float4 o;
    o.x = OP == 0 ? __fadd_rn(av.x, bv.x) : __fmul_rn(av.x, bv.x);
    o.y = OP == 0 ? __fadd_rn(av.y, bv.y) : __fmul_rn(av.y, bv.y);
    o.z = OP == 0 ? __fadd_rn(av.z, bv.z) : __fmul_rn(av.z, bv.z);
    o.w = OP == 0 ? __fadd_rn(av.w, bv.w) : __fmul_rn(av.w, bv.w);
    *reinterpret_cast<float4 *>(y + r * y_stride + c) = o;
}

int launch_binary(int op, const float *a, int64_t a_stride, const float *b, int64_t b_stride, int64_t b_ne0, int64_t b_rows,
                  float *y, int64_t y_stride, int64_t ne0, int64_t nrows, cudaStream_t s) {
    B200_REQUIRE(op == 0 || op == 1, "binary: op %d is neither add (0) nor mul (1)", op);
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30) && b_ne0 > 0 && ne0 % b_ne0 == 0 && b_rows > 0, "binary: operand shapes do not broadcast");
    const int64_t total = ne0 * nrows;
    if (total == 0) return B200_STATUS_SUCCESS;
    const auto al = [](const void *p, int64_t stride) { return ((uintptr_t)p & 15) == 0 && (stride & 3) == 0; };
    if (nrows > 1 && b_ne0 == ne0 && ne0 % 4 == 0 && al(a, a_stride) && al(b, b_stride) && al(y, y_stride)) {
        const int64_t total4 = total / 4, blocks4 = (total4 + 255) / 256;
        B200_REQUIRE(blocks4 < 0x7fffffffLL, "binary: tensor too large for one launch");
        if (op == 0)
            return launch_pdl(binary_vec_kernel<0>, dim3((unsigned)blocks4), dim3(256), 0, s, a, a_stride, b, b_stride, b_rows, y, y_stride,
                              (int)(ne0 / 4), total4);
        return launch_pdl(binary_vec_kernel<1>, dim3((unsigned)blocks4), dim3(256), 0, s, a, a_stride, b, b_stride, b_rows, y, y_stride,
                          (int)(ne0 / 4), total4);
    }
    const int64_t blocks = (total + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL, "binary: tensor too large for one launch");
    if (op == 0)
        return launch_pdl(binary_kernel<0>, dim3((unsigned)blocks), dim3(256), 0, s, a, a_stride, b, b_stride, (int)b_ne0, b_rows, y,
                          y_stride, (int)ne0, total);
    return launch_pdl(binary_kernel<1>, dim3((unsigned)blocks), dim3(256), 0, s, a, a_stride, b, b_stride, (int)b_ne0, b_rows, y,
                      y_stride, (int)ne0, total);
}

// ---- SILU (+ optional gate MUL) --------------------------------------------------------------------
// crates/ggml/src/simd_x86.rs:1012-1054: on a host with AVX512F+DQ the reference runs whole 16-lane
// chunks of a row through x / (1 + v_expf(0 - x)) and the remaining lanes through x / (1 + expf(-x))
// with the libm expf; on other hosts every lane takes the libm form.  wide selects which host is
// being reproduced.  With g != nullptr the kernel also emits silu(x) * g
// (crates/llama/src/graph_arch.rs:1150-1151).
__global__ void __launch_bounds__(256)
silu_kernel(const float *__restrict__ x, int64_t x_stride, const float *__restrict__ g, int64_t g_stride, float *y,
            int64_t y_stride, float *y_mul, int64_t y_mul_stride, int ne0, int wide_end, int64_t total) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / ne0;
    const int c = (int)(i - r * ne0);
    const float v = x[r * x_stride + c];
    const float e = c < wide_end ? v_expf(__fsub_rn(0.0f, v)) : libm_expf(-v);
    const float sv = __fdiv_rn(v, __fadd_rn(1.0f, e));
    if (y) y[r * y_stride + c] = sv;
    if (g) y_mul[r * y_mul_stride + c] = __fmul_rn(sv, g[r * g_stride + c]);
}

int launch_silu(const float *x, int64_t x_stride, const float *g, int64_t g_stride, float *y, int64_t y_stride, float *y_mul,
                int64_t y_mul_stride, int64_t ne0, int64_t nrows, int wide, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30), "silu: bad row length %lld", (long long)ne0);
    const int64_t total = ne0 * nrows;
    if (total == 0) return B200_STATUS_SUCCESS;
    const int64_t blocks = (total + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL, "silu: tensor too large for one launch");
    const int wide_end = wide ? (int)(ne0 & ~(int64_t)15) : 0;
    return launch_pdl(silu_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, x_stride, g, g_stride, y, y_stride, y_mul, y_mul_stride,
                      (int)ne0, wide_end, total);
}

// Few rows: the same, followed by the Q8_K quantization of the result (the gated product when g is given): grid
// (ne0 / 256, rows), one 256-element block per CTA.
__global__ void __launch_bounds__(256)
silu_q8_few_kernel(const float *__restrict__ x, int64_t x_stride, const float *__restrict__ g, int64_t g_stride, float *y,
               int64_t y_stride, float *y_mul, int64_t y_mul_stride, int wide_end, ActBuf act, int64_t m4) {
    pdl_trigger();
    pdl_wait();
    const int64_t r = blockIdx.y;
    const int c = blockIdx.x * 256 + threadIdx.x;
    const float v = x[r * x_stride + c];
    const float e = c < wide_end ? v_expf(__fsub_rn(0.0f, v)) : libm_expf(-v);
    const float sv = __fdiv_rn(v, __fadd_rn(1.0f, e));
    if (y) y[r * y_stride + c] = sv;
    float out = sv;
    if (g) {
        out = __fmul_rn(sv, g[r * g_stride + c]);
        y_mul[r * y_mul_stride + c] = out;
    }
    if (r < m4) q8_K_block_store<true>(out, act, r, blockIdx.x);
    else q8_K_block_store<false>(out, act, r, blockIdx.x);
}

// Many rows: one warp per
// 256-element block, lane l holding elements 8 l .. 8 l + 7 (16-byte loads and stores, no CTA barrier).
__global__ void __launch_bounds__(256)
silu_q8_kernel(const float *__restrict__ x, int64_t x_stride, const float *__restrict__ g, int64_t g_stride, float *y,
               int64_t y_stride, float *y_mul, int64_t y_mul_stride, int wide_end, int nblk, int64_t nwork, ActBuf act, int64_t m4, bool vec) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t wg = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wg >= nwork) return;
    const int64_t r = wg / nblk;
    const int blk = (int)(wg - r * nblk);
    const int c = blk * 256 + 8 * lane;
    float xs[8], v[8];
    load8(x + r * x_stride + c, vec, xs);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const float e = c + j < wide_end ? v_expf(__fsub_rn(0.0f, xs[j])) : libm_expf(-xs[j]);
        v[j] = __fdiv_rn(xs[j], __fadd_rn(1.0f, e));
    }
    if (y) store8(y + r * y_stride + c, vec, v);
    if (g) {
        float gs[8];
        load8(g + r * g_stride + c, vec, gs);
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = __fmul_rn(v[j], gs[j]);
        store8(y_mul + r * y_mul_stride + c, vec, v);
    }
    if (r < m4) q8_K_block_store_warp<true>(v, act, r, blk);
    else q8_K_block_store_warp<false>(v, act, r, blk);
}

int launch_silu_q8(const float *x, int64_t x_stride, const float *g, int64_t g_stride, float *y, int64_t y_stride, float *y_mul,
                   int64_t y_mul_stride, int64_t ne0, int64_t nrows, int wide, ActBuf act, int64_t m4, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 % 256 == 0 && ne0 < (1 << 30), "silu + q8_K: row length %lld is not a multiple of 256", (long long)ne0);
    const bool vec = aligned16(x, x_stride) && (!y || aligned16(y, y_stride)) && (!g || (aligned16(g, g_stride) && aligned16(y_mul, y_mul_stride)));
    if (nrows == 0) return B200_STATUS_SUCCESS;
    const int64_t nblk = ne0 / 256, nwork = nblk * nrows, blocks = (nwork + 7) / 8;
    B200_REQUIRE(blocks < 0x7fffffffLL, "silu + q8_K: tensor too large for one launch");
    const int wide_end = wide ? (int)(ne0 & ~(int64_t)15) : 0;
    if (nrows <= FEW_ROWS)
        return launch_pdl(silu_q8_few_kernel, dim3((unsigned)(ne0 / 256), (unsigned)nrows), dim3(256), 0, s, x, x_stride, g, g_stride, y, y_stride,
                          y_mul, y_mul_stride, wide_end, act, m4);
    return launch_pdl(silu_q8_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, x_stride, g, g_stride, y, y_stride, y_mul, y_mul_stride,
                      wide_end, (int)nblk, nwork, act, m4, vec);
}

// ---- ROPE --------------------------------------------------------------------------------------------
// The (cos, sin) table of crates/ggml/src/compute.rs:3520-3566 (rope_yarn, rope_cache_init) and :3627-3635
// (rope_yarn_corr_dims), computed on the host with the host's libm exactly as the reference computes it:
// table[t][i0] = cos(theta) * mscale, table[t][i0 + 1] = sin(theta) * mscale, theta walking the row in
// steps of theta_scale = powf(freq_base, -2 / n_dims) from the token's position.
static float rope_yarn_ramp(float low, float high, int64_t i0) {
    const float y = ((float)(i0 / 2) - low) / fmaxf(0.001f, high - low);
    return 1.0f - fminf(1.0f, fmaxf(0.0f, y));
}

void rope_table_host(const int32_t *pos, int64_t n_tok, int64_t ne0, const float *freq_factors, int n_dims, int n_ctx_orig,
                     float freq_base, float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow,
                     float *table) {
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    auto corr_dim = [&](float n_rot) {
        return (float)n_dims * logf((float)n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * logf(freq_base));
    };
    const float corr0 = fmaxf(0.0f, floorf(corr_dim(beta_fast)));
    const float corr1 = fminf((float)(n_dims - 1), ceilf(corr_dim(beta_slow)));
    for (int64_t t = 0; t < n_tok; t++) {
        float theta = (float)pos[t];
        float *c = table + t * ne0;
        for (int64_t i0 = 0; i0 + 1 < ne0; i0 += 2) {
            const float ff = freq_factors ? freq_factors[i0 / 2] : 1.0f;
            const float theta_extrap = theta / ff;
            const float theta_interp = freq_scale * theta_extrap;
            float th = theta_interp, mscale = attn_factor;
            if (ext_factor != 0.0f) {
                const float ramp_mix = rope_yarn_ramp(corr0, corr1, i0) * ext_factor;
                th = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
                mscale *= 1.0f + 0.1f * logf(1.0f / freq_scale);
            }
            c[i0] = cosf(th) * mscale;
            c[i0 + 1] = sinf(th) * mscale;
            theta *= theta_scale;
        }
    }
}

// crates/ggml/src/compute.rs:3663-3677 rotate_pairs_f32 and :3740-3775: one thread per channel pair of
// one head of one token.  Pairs inside n_dims rotate (adjacent channels in mode 0, channels n_dims/2
// apart in mode 2), the rest copy.  Token t reads row t of the table, or row rows[t] when the table holds
// one row per position; a row index outside the table skips the token and raises the error word.
__global__ void __launch_bounds__(256)
rope_kernel(const float *__restrict__ x, int64_t x_nb1, int64_t x_nb2, float *y, int64_t y_nb1, int64_t y_nb2,
            const float *__restrict__ table, const int32_t *__restrict__ rows, int64_t n_rows, int ne0, int n_head, int n_dims,
            int neox, int64_t total, int *err) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int half = ne0 / 2;
    const int p = (int)(i % half);
    const int64_t row = i / half;
    const int h = (int)(row % n_head);
    const int64_t t = row / n_head;
    const float *src = (const float *)((const char *)x + h * x_nb1 + t * x_nb2);
    float *dst = (float *)((char *)y + h * y_nb1 + t * y_nb2);
    const int i0 = 2 * p;
    const int64_t tr = rows ? (int64_t)rows[t] : t;
    if (tr < 0 || tr >= n_rows) {
        if (p == 0 && h == 0) atomicExch(err, 3);
        return;
    }
    if (i0 < n_dims) {
        const int ic = neox ? p : i0;
        const int off = neox ? n_dims / 2 : 1;
        const float c = table[tr * ne0 + i0], s = table[tr * ne0 + i0 + 1];
        const float x0 = src[ic], x1 = src[ic + off];
        dst[ic] = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
        dst[ic + off] = __fmaf_rn(x0, s, __fmul_rn(x1, c));
    } else {
        dst[i0] = src[i0];
        dst[i0 + 1] = src[i0 + 1];
    }
}

int launch_rope(const float *x, int64_t x_nb1, int64_t x_nb2, float *y, int64_t y_nb1, int64_t y_nb2, const float *table,
                const int32_t *rows, int64_t n_rows, int64_t ne0, int64_t n_head, int64_t n_tok, int n_dims, int mode, cudaStream_t s) {
    B200_REQUIRE(mode == 0 || mode == 2, "rope: mode %d is neither NORMAL (0) nor NEOX (2)", mode);
    B200_REQUIRE(ne0 > 0 && ne0 % 2 == 0 && n_dims > 0 && n_dims % 2 == 0 && n_dims <= ne0, "rope: bad head size %lld / n_dims %d",
                 (long long)ne0, n_dims);
    const int64_t total = n_tok * n_head * (ne0 / 2);
    if (total == 0) return B200_STATUS_SUCCESS;
    const int64_t blocks = (total + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL && n_head < (1 << 30) && ne0 < (1 << 30), "rope: tensor too large for one launch");
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_pdl(rope_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, x_nb1, x_nb2, y, y_nb1, y_nb2, table, rows,
                      rows ? n_rows : n_tok, (int)ne0, (int)n_head, n_dims, mode == 2 ? 1 : 0, total, err);
}

// ---- SET_ROWS into an F16 destination ----------------------------------------------------------------
// crates/ggml/src/compute.rs:4265-4338: row r of the f32 source goes, rounded to nearest even, to row
// idx[r] of the destination.  An index outside the destination is skipped and raises the error word.
__global__ void __launch_bounds__(256)
set_rows_f16_kernel(const float *__restrict__ x, int64_t x_stride, const int64_t *__restrict__ idx, __half *dst,
                    int64_t dst_stride, int64_t dst_rows, int ne0, int64_t total, int *err) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / ne0;
    const int c = (int)(i - r * ne0);
    const int64_t d = idx[r];
    if (d < 0 || d >= dst_rows) {
        if (c == 0) atomicExch(err, 2);
        return;
    }
    dst[d * dst_stride + c] = __float2half_rn(x[r * x_stride + c]);
}

int launch_set_rows_f16(const float *x, int64_t x_stride, const int64_t *idx, void *dst, int64_t dst_stride, int64_t dst_rows,
                        int64_t ne0, int64_t nrows, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30), "set_rows: bad row length %lld", (long long)ne0);
    const int64_t total = ne0 * nrows;
    if (total == 0) return B200_STATUS_SUCCESS;
    const int64_t blocks = (total + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL, "set_rows: tensor too large for one launch");
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_pdl(set_rows_f16_kernel, dim3((unsigned)blocks), dim3(256), 0, s, x, x_stride, idx, (__half *)dst, dst_stride,
                      dst_rows, (int)ne0, total, err);
}

// ---- several ROPE / SET_ROWS nodes in one launch ------------------------------------------------------
// At one token the attention block's glue is four kernels of a few thousand elements each: ROPE of K, SET_ROWS
// of K into the cache, SET_ROWS of V, ROPE of Q (crates/llama/src/graph_arch.rs:171-190, 1173-1240).  They are
// independent of one another once the SET_ROWS of K reads the rotated values straight from the ROPE that
// made them, so blockIdx.y walks up to four of them.  Element for element the arithmetic is rope_kernel's and
// set_rows_f16_kernel's: a ROPE with a cache attached stores the f32 result and its f16 rounding.
__global__ void __launch_bounds__(256)
glue_batch_kernel(GlueBatch b, int *err) {
    pdl_trigger();
    pdl_wait();
    const GlueOp &o = b.op[blockIdx.y];
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= o.total) return;
    if (o.kind == GLUE_SET_ROWS) {
        const int64_t r = i / o.ne0;
        const int c = (int)(i - r * o.ne0);
        const int64_t d = o.cache_idx[r];
        if (d < 0 || d >= o.cache_rows) {
            if (c == 0) atomicExch(err, 2);
            return;
        }
        ((__half *)o.cache)[d * o.cache_stride + c] = __float2half_rn(o.x[r * o.x_nb1 + c]);
        return;
    }
    const int half = o.ne0 / 2;
    const int p = (int)(i % half);
    const int64_t row = i / half;
    const int h = (int)(row % o.n_head);
    const int64_t t = row / o.n_head;
    const float *src = (const float *)((const char *)o.x + h * o.x_nb1 + t * o.x_nb2);
    float *dst = (float *)((char *)o.y + h * o.y_nb1 + t * o.y_nb2);
    const int i0 = 2 * p;
    const int64_t tr = o.rows ? (int64_t)o.rows[t] : t;
    if (tr < 0 || tr >= o.n_rows) {
        if (p == 0 && h == 0) atomicExch(err, 3);
        return;
    }
    float v0, v1;
    int e0, e1;
    if (i0 < o.n_dims) {
        e0 = o.neox ? p : i0;
        e1 = e0 + (o.neox ? o.n_dims / 2 : 1);
        const float c = o.table[tr * o.ne0 + i0], s = o.table[tr * o.ne0 + i0 + 1];
        const float x0 = src[e0], x1 = src[e1];
        v0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
        v1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
    } else {
        e0 = i0;
        e1 = i0 + 1;
        v0 = src[e0];
        v1 = src[e1];
    }
    dst[e0] = v0;
    dst[e1] = v1;
    if (o.cache) {
        const int64_t d = o.cache_idx[t];
        if (d < 0 || d >= o.cache_rows) {
            if (p == 0 && h == 0) atomicExch(err, 2);
            return;
        }
        __half *crow = (__half *)o.cache + d * o.cache_stride + (int64_t)h * o.ne0;
        crow[e0] = __float2half_rn(v0);
        crow[e1] = __float2half_rn(v1);
    }
}

int launch_glue_batch(const GlueBatch &b, cudaStream_t s) {
    B200_REQUIRE(b.count >= 1 && b.count <= GLUE_BATCH_MAX, "glue batch: %d operations", b.count);
    int64_t most = 0;
    for (int i = 0; i < b.count; i++) {
        const GlueOp &o = b.op[i];
        B200_REQUIRE(o.kind == GLUE_ROPE || o.kind == GLUE_SET_ROWS, "glue batch: operation %d has kind %d", i, o.kind);
        B200_REQUIRE(o.ne0 > 0 && o.total >= 0, "glue batch: operation %d has a bad shape", i);
        if (o.kind == GLUE_ROPE)
            B200_REQUIRE(o.ne0 % 2 == 0 && o.n_dims > 0 && o.n_dims % 2 == 0 && o.n_dims <= o.ne0 && o.n_head > 0, "glue batch: bad rope shape");
        most = o.total > most ? o.total : most;
    }
    if (most == 0) return B200_STATUS_SUCCESS;
    const int64_t blocks = (most + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL, "glue batch: tensor too large for one launch");
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_pdl(glue_batch_kernel, dim3((unsigned)blocks, (unsigned)b.count), dim3(256), 0, s, b, err);
}

// ---- GET_ROWS from F32 / F16 tables ------------------------------------------------------------------
// crates/ggml/src/compute.rs:3842-3895 (the quantized tables go through get_rows_tiled_kernel).
template <typename T>
__global__ void __launch_bounds__(256)
get_rows_plain_kernel(const T *__restrict__ table, int64_t table_stride, int64_t table_rows, const int32_t *__restrict__ ids,
                      float *out, int64_t out_stride, int ne0, int64_t total, int *err) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t r = i / ne0;
    const int c = (int)(i - r * ne0);
    const int64_t row = ids[r];
    if (row < 0 || row >= table_rows) {
        if (c == 0) atomicExch(err, 1);
        return;
    }
    out[r * out_stride + c] = (float)table[row * table_stride + c];
}

int launch_get_rows(int type, const void *table, int64_t ne0, int64_t table_rows, const int32_t *ids, int64_t n, float *out,
                    int64_t out_stride, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30), "get_rows: bad row length %lld", (long long)ne0);
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (is_quant_type(type)) return launch_get_rows_tiled(type, table_rows, ne0, (const uint8_t *)table, ids, n, out, out_stride, err, s);
    B200_REQUIRE(type == B200_TYPE_F32 || type == B200_TYPE_F16, "get_rows: table type %d is not supported", type);
    const int64_t total = ne0 * n;
    if (total == 0) return B200_STATUS_SUCCESS;
    const int64_t blocks = (total + 255) / 256;
    B200_REQUIRE(blocks < 0x7fffffffLL, "get_rows: too many rows for one launch");
    if (type == B200_TYPE_F32)
        return launch_pdl(get_rows_plain_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, s, (const float *)table, ne0, table_rows,
                          ids, out, out_stride, (int)ne0, total, err);
    return launch_pdl(get_rows_plain_kernel<__half>, dim3((unsigned)blocks), dim3(256), 0, s, (const __half *)table, ne0, table_rows, ids,
                      out, out_stride, (int)ne0, total, err);
}

// ---- ARGMAX --------------------------------------------------------------------------------------------
// crates/ggml/src/compute.rs:4208-4228: the largest element of each row, the last one among equals;
// a row of NaNs or of -inf gives the reference's answers too (max stays -inf; the last -inf matches).
__global__ void __launch_bounds__(1024)
argmax_kernel(const float *__restrict__ x, int64_t x_stride, int32_t *out, int ne0) {
    pdl_trigger();
    pdl_wait();
    const float *xr = x + (int64_t)blockIdx.x * x_stride;
    float best = -INFINITY;
    int at = -1;   // -1: nothing equal to the running maximum seen yet
    // (value, index) pairs merge the same way in any order (larger value, then larger index), so the row is
    // read with 16-byte loads, several in flight per thread, when its length and address allow
    auto take = [&](float v, int i) {
        if (v > best) { best = v; at = i; }
        else if (v == best && i > at) at = i;
    };
    if ((ne0 & 3) == 0 && (((uintptr_t)xr) & 15) == 0) {
        const float4 *x4 = (const float4 *)xr;
        const int n4 = ne0 >> 2;
#pragma unroll 4
        for (int i = threadIdx.x; i < n4; i += 1024) {
            const float4 v = x4[i];
            take(v.x, 4 * i);
            take(v.y, 4 * i + 1);
            take(v.z, 4 * i + 2);
            take(v.w, 4 * i + 3);
        }
    } else {
        for (int i = threadIdx.x; i < ne0; i += 1024) take(xr[i], i);
    }
    __shared__ float sb[32];
    __shared__ int sa[32];
    auto merge = [](float &b, int &a, float ob, int oa) {
        if (ob > b || (ob == b && oa > a)) { b = ob; a = oa; }
    };
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        merge(best, at, ob, oa);
    }
    if ((threadIdx.x & 31) == 0) { sb[threadIdx.x >> 5] = best; sa[threadIdx.x >> 5] = at; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sb[threadIdx.x];
        at = sa[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            merge(best, at, ob, oa);
        }
        if (threadIdx.x == 0) out[blockIdx.x] = at < 0 ? 0 : at;
    }
}

int launch_argmax(const float *x, int64_t x_stride, int64_t ne0, int64_t nrows, int32_t *out, cudaStream_t s) {
    B200_REQUIRE(ne0 > 0 && ne0 < (1 << 30) && nrows < 0x7fffffffLL, "argmax: bad shape");
    if (nrows == 0) return B200_STATUS_SUCCESS;
    return launch_pdl(argmax_kernel, dim3((unsigned)nrows), dim3(1024), 0, s, x, x_stride, out, (int)ne0);
}

}  // namespace b200

// ---- C ABI ---------------------------------------------------------------------------------------------
using namespace b200;

extern "C" {

int b200_rms_norm(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *weight, float *y_weighted,
                  int64_t y_weighted_stride, int64_t ne0, int64_t nrows, float eps, void *stream) {
    B200_REQUIRE(x != nullptr && (y != nullptr || (weight != nullptr && y_weighted != nullptr)), "rms_norm: null operand");
    B200_REQUIRE(weight == nullptr || y_weighted != nullptr, "rms_norm: weight given without y_weighted");
    return launch_rms_norm(x, x_stride, y, y_stride, weight, y_weighted, y_weighted_stride, ne0, nrows, eps, (cudaStream_t)stream);
}

// rows below m4 of a MIXED result take the 4x8 value rule: what the Q4_K 8x8 route reads (see b200_act_quant)
static int q8_K_rows_4x8(int act_kind, int64_t nrows, int64_t *m4) {
    B200_REQUIRE(act_kind == B200_ACT_Q8_K || act_kind == B200_ACT_Q8_K_4X8 || act_kind == B200_ACT_Q8_K_MIXED,
                 "fused quantization supports the Q8_K kinds only (kind %d)", act_kind);
    *m4 = act_kind == B200_ACT_Q8_K ? 0 : act_kind == B200_ACT_Q8_K_4X8 ? nrows : nrows - nrows % 4;
    return B200_STATUS_SUCCESS;
}

int b200_rms_norm_q8(const float *x, int64_t x_stride, float *y, int64_t y_stride, const float *weight, float *y_weighted,
                     int64_t y_weighted_stride, int64_t ne0, int64_t nrows, float eps, void *dev_act, int act_kind, void *stream) {
    B200_REQUIRE(x != nullptr && dev_act != nullptr, "rms_norm_q8: null operand");
    B200_REQUIRE(weight == nullptr || y_weighted != nullptr, "rms_norm_q8: weight given without y_weighted");
    B200_REQUIRE(((uintptr_t)dev_act & 255) == 0, "rms_norm_q8: scratch must be 256-byte aligned");
    int64_t m4 = 0;
    int rc = q8_K_rows_4x8(act_kind, nrows, &m4);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_rms_norm_q8(x, x_stride, y, y_stride, weight, y_weighted, y_weighted_stride, ne0, nrows, eps,
                              act_carve(dev_act, nrows, ne0), m4, (cudaStream_t)stream);
}

int b200_binary(int op, const float *a, int64_t a_stride, const float *b, int64_t b_stride, int64_t b_ne0, int64_t b_rows, float *y,
                int64_t y_stride, int64_t ne0, int64_t nrows, void *stream) {
    B200_REQUIRE(a != nullptr && b != nullptr && y != nullptr, "binary: null operand");
    return launch_binary(op, a, a_stride, b, b_stride, b_ne0, b_rows, y, y_stride, ne0, nrows, (cudaStream_t)stream);
}

int b200_silu(const float *x, int64_t x_stride, const float *gate, int64_t gate_stride, float *y, int64_t y_stride, float *y_gated,
              int64_t y_gated_stride, int64_t ne0, int64_t nrows, int wide, void *stream) {
    B200_REQUIRE(x != nullptr && (y != nullptr || (gate != nullptr && y_gated != nullptr)), "silu: null operand");
    B200_REQUIRE(gate == nullptr || y_gated != nullptr, "silu: gate given without y_gated");
    return launch_silu(x, x_stride, gate, gate_stride, y, y_stride, y_gated, y_gated_stride, ne0, nrows, wide, (cudaStream_t)stream);
}

int b200_silu_q8(const float *x, int64_t x_stride, const float *gate, int64_t gate_stride, float *y, int64_t y_stride, float *y_gated,
                 int64_t y_gated_stride, int64_t ne0, int64_t nrows, int wide, void *dev_act, int act_kind, void *stream) {
    B200_REQUIRE(x != nullptr && dev_act != nullptr, "silu_q8: null operand");
    B200_REQUIRE(gate == nullptr || y_gated != nullptr, "silu_q8: gate given without y_gated");
    B200_REQUIRE(((uintptr_t)dev_act & 255) == 0, "silu_q8: scratch must be 256-byte aligned");
    int64_t m4 = 0;
    int rc = q8_K_rows_4x8(act_kind, nrows, &m4);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_silu_q8(x, x_stride, gate, gate_stride, y, y_stride, y_gated, y_gated_stride, ne0, nrows, wide,
                          act_carve(dev_act, nrows, ne0), m4, (cudaStream_t)stream);
}

int b200_host_silu_is_wide(void) { return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512dq") ? 1 : 0; }

int b200_rope_table(const int32_t *pos, int64_t n_tok, int64_t ne0, const float *freq_factors, int n_dims, int n_ctx_orig,
                    float freq_base, float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow,
                    float *table) {
    B200_REQUIRE(pos != nullptr && table != nullptr, "rope_table: null operand");
    B200_REQUIRE(ne0 > 0 && ne0 % 2 == 0 && n_dims > 0 && n_dims % 2 == 0 && n_dims <= ne0, "rope_table: bad head size %lld / n_dims %d",
                 (long long)ne0, n_dims);
    rope_table_host(pos, n_tok, ne0, freq_factors, n_dims, n_ctx_orig, freq_base, freq_scale, ext_factor, attn_factor, beta_fast,
                    beta_slow, table);
    return B200_STATUS_SUCCESS;
}

int b200_rope(const float *x, int64_t x_nb1, int64_t x_nb2, float *y, int64_t y_nb1, int64_t y_nb2, const float *table,
              const int32_t *table_rows, int64_t table_n_rows, int64_t ne0, int64_t n_head, int64_t n_tok, int n_dims, int mode,
              void *stream) {
    B200_REQUIRE(x != nullptr && y != nullptr && table != nullptr, "rope: null operand");
    B200_REQUIRE(x_nb1 % 4 == 0 && x_nb2 % 4 == 0 && y_nb1 % 4 == 0 && y_nb2 % 4 == 0, "rope: strides must be multiples of 4 bytes");
    B200_REQUIRE(table_rows == nullptr || table_n_rows > 0, "rope: a row index needs the table's row count");
    return launch_rope(x, x_nb1, x_nb2, y, y_nb1, y_nb2, table, table_rows, table_n_rows, ne0, n_head, n_tok, n_dims, mode,
                       (cudaStream_t)stream);
}

int b200_set_rows_f16(const float *x, int64_t x_stride, const int64_t *idx, void *dst, int64_t dst_stride, int64_t dst_rows,
                      int64_t ne0, int64_t nrows, void *stream) {
    B200_REQUIRE(x != nullptr && idx != nullptr && dst != nullptr, "set_rows: null operand");
    return launch_set_rows_f16(x, x_stride, idx, dst, dst_stride, dst_rows, ne0, nrows, (cudaStream_t)stream);
}

int b200_get_rows(int type, const void *table, int64_t ne0, int64_t table_rows, const int32_t *ids, int64_t n, float *y,
                  int64_t y_stride, void *stream) {
    B200_REQUIRE(table != nullptr && ids != nullptr && y != nullptr, "get_rows: null operand");
    return launch_get_rows(type, table, ne0, table_rows, ids, n, y, y_stride, (cudaStream_t)stream);
}

int b200_argmax(const float *x, int64_t x_stride, int64_t ne0, int64_t nrows, int32_t *out, void *stream) {
    B200_REQUIRE(x != nullptr && out != nullptr, "argmax: null operand");
    return launch_argmax(x, x_stride, ne0, nrows, out, (cudaStream_t)stream);
}

}  // extern "C"
