// On-the-fly Q8 quantization of f32 activation rows, bit-exact with the CPU
// path's three value rules:
//   A1 quantize_row_q8_0      crates/ggml/src/quants.rs:331-362
//   A2 quantize_row_q8_K      crates/ggml/src/quants.rs:615-654
//   A3 quantize_mat_q8_K_4x8  crates/ggml/src/repack.rs:1561-1606 (values; the
//      4-row interleaved storage is a CPU detail, the device keeps plain rows)
// Every float op is an explicit round-to-nearest intrinsic: no FMA contraction.
#include "common.cuh"
#include "act_quant.cuh"

namespace b200 {

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t act_scratch_bytes(int64_t m, int64_t k) {
    size_t b = 0;
    b += align_up((size_t)m * k, 256);            // qs
    b += align_up((size_t)m * (k / 256) * 4, 256);  // d
    b += align_up((size_t)m * (k / 16) * 2, 256);   // bsums
    b += align_up((size_t)m * (k / 32) * 2, 256);   // dh
    return b;
}

ActBuf act_carve(void *scratch, int64_t m, int64_t k) {
    uint8_t *p = (uint8_t *)scratch;
    ActBuf a;
    a.k = k;
    a.qs = (int8_t *)p;
    p += align_up((size_t)m * k, 256);
    a.d = (float *)p;
    p += align_up((size_t)m * (k / 256) * 4, 256);
    a.bsums = (int16_t *)p;
    p += align_up((size_t)m * (k / 16) * 2, 256);
    a.dh = (uint16_t *)p;
    return a;
}

// A2 / A3: one CTA of 256 threads per (256-element block, row); the block's arithmetic is q8_K_block_store
// (act_quant.cuh), shared with the kernels that quantize what they have just computed.
template <bool A3>
__global__ void __launch_bounds__(256) quantize_q8_K_kernel(const float *__restrict__ x, int64_t ldx, ActBuf out) {
    pdl_trigger();
    pdl_wait();   // x comes from the previous kernel; the scratch written here may still be read by it
    const int64_t blk = blockIdx.x, row = blockIdx.y;
    q8_K_block_store<A3>(x[row * ldx + blk * 256 + threadIdx.x], out, row, blk);
}

// The same for prompt batches (more than 32 rows): one warp per block, lane l holding elements 8 l .. 8 l + 7, no
// CTA barrier (q8_K_block_store_warp); 16-byte loads when the rows allow it.
template <bool A3>
__global__ void __launch_bounds__(256) quantize_q8_K_rows_kernel(const float *__restrict__ x, int64_t ldx, ActBuf out, int nblk, int64_t nwork, bool vec) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t wg = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wg >= nwork) return;
    const int64_t row = wg / nblk, blk = wg - row * nblk;
    const float *p = x + row * ldx + blk * 256 + 8 * lane;
    float v[8];
    if (vec) {
        const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = p[j];
    }
    q8_K_block_store_warp<A3>(v, out, row, blk);
}

template <bool A3>
static int launch_q8_K(int64_t m, int64_t k, const float *x, int64_t ldx, ActBuf out, cudaStream_t s) {
    if (m <= 32) return launch_pdl(quantize_q8_K_kernel<A3>, dim3((unsigned)(k / 256), (unsigned)m), dim3(256), 0, s, x, ldx, out);
    const int64_t nblk = k / 256, nwork = nblk * m, blocks = (nwork + 7) / 8;
    B200_REQUIRE(blocks < 0x7fffffffLL, "quantize q8_K: tensor too large for one launch");
    const bool vec = ((uintptr_t)x & 15) == 0 && ldx % 4 == 0;
    return launch_pdl(quantize_q8_K_rows_kernel<A3>, dim3((unsigned)blocks), dim3(256), 0, s, x, ldx, out, (int)nblk, nwork, vec);
}

// A1: one warp per 32-element block, 8 blocks per CTA.
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, int64_t ldx, ActBuf out) {
    pdl_trigger();
    pdl_wait();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int64_t row = blockIdx.y;
    const int64_t blk = (int64_t)blockIdx.x * 8 + warp;
    if (blk >= out.k / 32) return;
    const float v = x[row * ldx + blk * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = amax != 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const float r = rintf(__fmul_rn(v, id));
    int q;
    if (isnan(r) || fabsf(r) >= 2147483648.0f) q = -128;  // the AVX2 cvt/packs saturation
    else q = max(-128, min(127, (int)r));
    out.qs[row * out.k + blk * 32 + lane] = (int8_t)q;
    if (lane == 0) out.dh[row * (out.k / 32) + blk] = __half_as_ushort(__float2half_rn(d));
}

int launch_quantize_acts(int kind, int64_t m, int64_t k, const float *x, int64_t ldx, ActBuf out, cudaStream_t s) {
    B200_REQUIRE(m >= 0 && m <= 65535, "quantize: %lld activation rows exceed one launch (max 65535)", (long long)m);
    if (m == 0) return B200_STATUS_SUCCESS;
    if (kind == B200_ACT_Q8_0) {
        B200_REQUIRE(k > 0 && k % 32 == 0, "quantize q8_0: k = %lld must be a positive multiple of 32", (long long)k);
        dim3 grid((unsigned)((k / 32 + 7) / 8), (unsigned)m);
        return launch_pdl(quantize_q8_0_kernel, grid, dim3(256), 0, s, x, ldx, out);
    } else if (kind == B200_ACT_Q8_K || kind == B200_ACT_Q8_K_4X8) {
        B200_REQUIRE(k > 0 && k % 256 == 0, "quantize q8_K: k = %lld must be a positive multiple of 256", (long long)k);
        if (kind == B200_ACT_Q8_K) return launch_q8_K<false>(m, k, x, ldx, out, s);
        return launch_q8_K<true>(m, k, x, ldx, out, s);
    } else if (kind == B200_ACT_Q8_K_MIXED) {
        B200_REQUIRE(k > 0 && k % 256 == 0, "quantize q8_K: k = %lld must be a positive multiple of 256", (long long)k);
        const int64_t m4 = m - m % 4;
        if (m4 > 0) {
            int rc = launch_q8_K<true>(m4, k, x, ldx, out, s);
            if (rc != B200_STATUS_SUCCESS) return rc;
        }
        if (m > m4) {
            ActBuf tail = out;
            tail.qs += m4 * k;
            tail.d += m4 * (k / 256);
            tail.bsums += m4 * (k / 16);
            int rc = launch_q8_K<false>(m - m4, k, x + m4 * ldx, ldx, tail, s);
            if (rc != B200_STATUS_SUCCESS) return rc;
        }
    } else {
        B200_REQUIRE(false, "quantize: unknown activation kind %d", kind);
    }
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

}  // namespace b200
