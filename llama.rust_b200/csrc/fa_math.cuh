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

__device__ __forceinline__ float libm_expf(float x) {
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
    unsigned long long t = (unsigned long long)__double_as_longlong(c_exp2_tab[ki & 31]);
    t += (ki >> 5) << 52;   // == T[ki % N] + (ki << 47) with the table's own bias folded out
    const double s = __longlong_as_double((long long)t);
    z = __fma_rn(c0, r, c1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(c2, r, 1.0);
    y = __fma_rn(z, r2, y);
    y = __dmul_rn(y, s);
    return __double2float_rn(y);
}

}  // namespace b200
