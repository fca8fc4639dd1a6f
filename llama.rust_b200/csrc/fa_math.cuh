// Device math shared by the attention kernels.
#pragma once
#include "common.cuh"

namespace b200 {

// ---------------------------------------------------------------------------
// expf as the host libm computes it (x86-64 glibc, FMA variant): N = 32 table,
// cubic in double precision.  Inputs here are <= 0 or small.
// ---------------------------------------------------------------------------
static __device__ const double c_exp2_tab[32] = {
    0x1.0000000000000p+0, 0x1.059b0d3158574p+0, 0x1.0b5586cf9890fp+0, 0x1.11301d0125b51p+0,
    0x1.172b83c7d517bp+0, 0x1.1d4873168b9aap+0, 0x1.2387a6e756238p+0, 0x1.29e9df51fdee1p+0,
    0x1.306fe0a31b715p+0, 0x1.371a7373aa9cbp+0, 0x1.3dea64c123422p+0, 0x1.44e086061892dp+0,
    0x1.4bfdad5362a27p+0, 0x1.5342b569d4f82p+0, 0x1.5ab07dd485429p+0, 0x1.6247eb03a5585p+0,
    0x1.6a09e667f3bcdp+0, 0x1.71f75e8ec5f74p+0, 0x1.7a11473eb0187p+0, 0x1.82589994cce13p+0,
    0x1.8ace5422aa0dbp+0, 0x1.93737b0cdc5e5p+0, 0x1.9c49182a3f090p+0, 0x1.a5503b23e255dp+0,
    0x1.ae89f995ad3adp+0, 0x1.b7f76f2fb5e47p+0, 0x1.c199bdd85529cp+0, 0x1.cb720dcef9069p+0,
    0x1.d5818dcfba487p+0, 0x1.dfc97337b9b5fp+0, 0x1.ea4afa2a490dap+0, 0x1.f50765b6e4540p+0};

__device__ __forceinline__ float libm_expf_tab(float x, const double *tab) {
    if (x != x) return x;
    if (x < -0x1.9fe368p6f) return 0.0f;                 // below log(2^-150)
    if (x > 0x1.62e42ep6f) return __int_as_float(0x7f800000);
    const double N = 32.0;
    const double invln2n = 0x1.71547652b82fep+0 * N;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / N / N / N, c1 = 0x1.ebfce50fac4f3p-3 / N / N, c2 = 0x1.62e42ff0c52d6p-1 / N;
    double z = __dmul_rn(invln2n, (double)x);
    double kd = __dadd_rn(z, shift);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, shift);
    const double r = __dsub_rn(z, kd);
    unsigned long long t = (unsigned long long)__double_as_longlong(tab[ki & 31]);
    t += (ki >> 5) << 52;   // == T[ki % N] + (ki << 47) with the table's own bias folded out
    const double s = __longlong_as_double((long long)t);
    z = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(z, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

__device__ __forceinline__ float libm_expf(float x) { return libm_expf_tab(x, c_exp2_tab); }

// one lane of ggml_v_expf (AVX512F+DQ branch): crates/ggml/src/flash_attn.rs:948-975
__device__ __forceinline__ float v_expf(float x) {
    const float R = __uint_as_float(0x4b400000u), LOG2E = __uint_as_float(0x3fb8aa3bu);
    const float C1 = __uint_as_float(0x35bfbe8eu), C2 = __uint_as_float(0x3f317200u);
    const float P1 = __uint_as_float(0x3c072010u), P2 = __uint_as_float(0x3d2b9f17u), P3 = __uint_as_float(0x3e2aaf33u);
    const float P4 = __uint_as_float(0x3efffedbu), P5 = __uint_as_float(0x3f7ffff6u);
    const float z = __fmaf_rn(x, LOG2E, R);
    const float n = __fsub_rn(z, R);
    const float b = __fmaf_rn(n, -C1, __fmaf_rn(n, -C2, x));
    const float u = __fmul_rn(b, b);
    const float j = __fmaf_rn(__fmaf_rn(__fmaf_rn(b, P1, P2), u, __fmaf_rn(b, P3, P4)), u, __fmaf_rn(b, P5, 1.0f));
    if (fabsf(n) > 192.0f) return n <= 0.0f ? 0.0f : __int_as_float(0x7f800000);
    return __double2float_rn(scalbn((double)j, (int)n));   // j * 2^n, rounded once
}

}  // namespace b200
