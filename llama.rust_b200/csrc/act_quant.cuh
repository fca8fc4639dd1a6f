// The Q8_K block quantizer as a device function, for kernels that quantize the 256 values a CTA holds.
#pragma once
#include "common.cuh"

namespace b200 {

// All 256 threads of the CTA call this with their value v = element threadIdx.x of block `blk` of
// activation row `row`.  A3 = false: quantize_row_q8_K (crates/ggml/src/quants.rs:615-654: the first
// largest |v| sets the sign of the scale, nearest_int); A3 = true: the 4x8 rule of
// crates/ggml/src/repack.rs:1561-1606 (scale 127 / amax, round to nearest even, clamp).
template <bool A3>
__device__ __forceinline__ void q8_K_block_store(float v, const ActBuf &out, int64_t row, int64_t blk) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int64_t nb = out.k / 256;
    __shared__ float s_a[8];
    __shared__ int s_i[8];
    __shared__ float s_x[256];
    s_x[t] = v;
    // largest |v|, first index on ties (the CPU scans with a strict '>')
    float a = fabsf(v);
    int idx = t;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float a2 = __shfl_xor_sync(0xffffffffu, a, o);
        int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (a2 > a || (a2 == a && i2 < idx)) { a = a2; idx = i2; }
    }
    if (lane == 0) { s_a[warp] = a; s_i[warp] = idx; }
    __syncthreads();
    a = s_a[0];
    idx = s_i[0];
#pragma unroll
    for (int w = 1; w < 8; w++) {
        float a2 = s_a[w];
        if (a2 > a) { a = a2; idx = s_i[w]; }  // later warps have larger indices: strict '>' keeps the first
    }
    const float amax = a;
    const float maxv = s_x[idx];
    int q = 0;
    float d = 0.0f;
    if (amax != 0.0f) {
        if (A3) {
            const float iscale = __fdiv_rn(127.0f, amax);
            q = __float2int_rn(__fmul_rn(iscale, v));  // round to nearest even
            q = max(-128, min(127, q));
            d = __fdiv_rn(1.0f, iscale);
        } else {
            const float iscale = __fdiv_rn(-127.0f, maxv);
            // nearest_int(): crates/ggml/src/quants.rs:13-18
            const float val = __fadd_rn(__fmul_rn(iscale, v), 12582912.0f);
            q = (__float_as_int(val) & 0x007fffff) - 0x00400000;
            q = min(127, q);
            d = __fdiv_rn(1.0f, iscale);
        }
    }
    out.qs[row * out.k + blk * 256 + t] = (int8_t)q;
    int s = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((t & 15) == 0) out.bsums[row * (out.k / 16) + blk * 16 + (t >> 4)] = (int16_t)s;
    if (t == 0) out.d[row * nb + blk] = d;
    __syncthreads();   // the shared arrays may be reused by a following call
}

// The same block handled by one warp: lane l holds elements 8 l .. 8 l + 7 of the 256.  No shared memory and no
// CTA barrier: warps of a CTA work on different blocks.  Same values as q8_K_block_store: the first largest |v|
// in index order, the same scale and rounding rules.
template <bool A3>
__device__ __forceinline__ void q8_K_block_store_warp(const float (&v)[8], const ActBuf &out, int64_t row, int64_t blk) {
    const int lane = threadIdx.x & 31;
    const int64_t nb = out.k / 256;
    float a = fabsf(v[0]), mv = v[0];
    int idx = 8 * lane;
#pragma unroll
    for (int j = 1; j < 8; j++) {
        const float aj = fabsf(v[j]);
        if (aj > a) { a = aj; mv = v[j]; idx = 8 * lane + j; }   // strict '>': the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float a2 = __shfl_xor_sync(0xffffffffu, a, o), m2 = __shfl_xor_sync(0xffffffffu, mv, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (a2 > a || (a2 == a && i2 < idx)) { a = a2; mv = m2; idx = i2; }
    }
    const float amax = a, maxv = mv;
    int q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float d = 0.0f;
    if (amax != 0.0f) {
        if (A3) {
            const float iscale = __fdiv_rn(127.0f, amax);
#pragma unroll
            for (int j = 0; j < 8; j++) q[j] = max(-128, min(127, __float2int_rn(__fmul_rn(iscale, v[j]))));
            d = __fdiv_rn(1.0f, iscale);
        } else {
            const float iscale = __fdiv_rn(-127.0f, maxv);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                // nearest_int(): crates/ggml/src/quants.rs:13-18
                const float val = __fadd_rn(__fmul_rn(iscale, v[j]), 12582912.0f);
                q[j] = min(127, (__float_as_int(val) & 0x007fffff) - 0x00400000);
            }
            d = __fdiv_rn(1.0f, iscale);
        }
    }
    uint2 packed;
    packed.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2 *>(out.qs + row * out.k + blk * 256 + 8 * lane) = packed;
    int s = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
    s += __shfl_xor_sync(0xffffffffu, s, 1);   // a 16-element sum is two lanes
    if ((lane & 1) == 0) out.bsums[row * (out.k / 16) + blk * 16 + (lane >> 1)] = (int16_t)s;
    if (lane == 0) out.d[row * nb + blk] = d;
}

// quantize_row_q8_K (the plain rule) on the block a warp holds in registers, lane l: elements 8 l .. 8 l + 7.  Returns
// the lane's eight quants packed in element order, the block scale d, and the sum of the lane's eight quants (two
// lanes make one of the block's 16-element sums).  Same values as q8_K_block_store_warp<false>.
__device__ __forceinline__ void q8_K_block_regs(const float (&v)[8], uint2 *packed, float *d_out, int *sum8) {
    const int lane = threadIdx.x & 31;
    float a = fabsf(v[0]), mv = v[0];
    int idx = 8 * lane;
#pragma unroll
    for (int j = 1; j < 8; j++) {
        const float aj = fabsf(v[j]);
        if (aj > a) { a = aj; mv = v[j]; idx = 8 * lane + j; }   // strict '>': the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float a2 = __shfl_xor_sync(0xffffffffu, a, o), m2 = __shfl_xor_sync(0xffffffffu, mv, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, idx, o);
        if (a2 > a || (a2 == a && i2 < idx)) { a = a2; mv = m2; idx = i2; }
    }
    int q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float d = 0.0f;
    if (a != 0.0f) {
        const float iscale = __fdiv_rn(-127.0f, mv);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            // nearest_int(): crates/ggml/src/quants.rs:13-18
            const float val = __fadd_rn(__fmul_rn(iscale, v[j]), 12582912.0f);
            q[j] = min(127, (__float_as_int(val) & 0x007fffff) - 0x00400000);
        }
        d = __fdiv_rn(1.0f, iscale);
    }
    packed->x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    packed->y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *d_out = d;
    *sum8 = q[0] + q[1] + q[2] + q[3] + q[4] + q[5] + q[6] + q[7];
}

}  // namespace b200
