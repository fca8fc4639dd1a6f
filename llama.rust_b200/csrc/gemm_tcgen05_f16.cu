// Q4_K prompt mat-mul, 8x8 gemm chain, with the sub-block scales folded into f16 tensor-core operands:
// 128 weight rows x 64 activation rows per CTA, half a super-block (two sub-block pairs) per pipeline step.
//
// Arithmetic (see gemm_tcgen05.cu for the argument): the gemm route needs, per sub-block pair g, the integers
//     ig = s_lo dot_lo + s_hi dot_hi  (< 2^23)      mg = m_lo bsum_lo + m_hi bsum_hi  (< 2^19)
// as f32.  With operands  s * w  (<= 945), the activation bytes, the mins and the 16-element activation sums
// (<= 2032), all exact in f16, and every partial sum an integer below 2^24, an f16 x f16 -> f32 MMA returns
// exactly f32(ig) and f32(mg); the epilogue is the chain's two fused multiply-adds per pair,
//     sumf = fma(f32(ig), d d_x, sumf);  summin = fma(f32(mg), dmin d_x, summin);  out = sumf - summin
// (crates/ggml/src/repack.rs:1692-1768), so the bits are those of the integer kernels and of the CPU.
//
// Shape of the pipeline, chosen from measurements of the 32-column / whole-super-block version: the A
// conversion and its shared-memory traffic are amortised over 64 columns, a step is half a super-block so that
// three 56 KB operand stages fit (tensor memory: two accumulator stages of 2 pairs x (ig, mg) x 64 columns),
// and all 16 worker warps do the same things in the same order - convert their share of step h into the free
// stage, hand it to the MMA warp, drain the accumulators of step h - 1 - so that they meet at every hand-off
// instead of polling for one another.
//   A  [128 rows][128 f16]  s * w;  K order within a pair: 16-byte piece p, (low | high) nibbles, bytes (0,2,1,3 ..)
//   B  [64 columns][128 f16] activation bytes in the same order
//   Am [128 rows][16 f16]   slots 4g, 4g+1 = m_lo of pair g, 4g+2, 4g+3 = m_hi (all four pairs of the super-block)
//   Bm [2 pairs][64 columns][16 f16]  slots 4g .. 4g+3 = the pair's four 16-element activation sums, rest 0
// K-major, no swizzle: 8 rows x 16 bytes core matrices, K-adjacent ones 128 bytes apart.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag and the device error word.
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int FX_ROWS = 128, FX_COLS = 64;
constexpr int FX_WORK_WARPS = 16;
constexpr int FX_THREADS = (FX_WORK_WARPS + 1) * 32;
constexpr int FX_STAGES = 3, FX_TSTAGES = 2;
constexpr int FX_A_BYTES = FX_ROWS * 256;          // 128 f16 per row
constexpr int FX_B_BYTES = FX_COLS * 256;
constexpr int FX_AM_BYTES = FX_ROWS * 32;
constexpr int FX_BM_BYTES = 2 * FX_COLS * 32;
constexpr int FX_STAGE_BYTES = FX_A_BYTES + FX_B_BYTES + FX_AM_BYTES + FX_BM_BYTES;   // 57344
constexpr int FX_SMEM_BYTES = FX_STAGES * FX_STAGE_BYTES + 1024;
constexpr int FX_DA_SLOTS = 4;
constexpr uint32_t FX_WAIT_LIMIT = 1u << 22;
constexpr int FX_ERR_WAIT = 4;
// kind::f16 instruction descriptor: f32 accumulator, f16 x f16, both operands K-major, N = 64, M = 128
constexpr uint32_t FX_IDESC = (1u << 4) | ((uint32_t)(FX_COLS >> 3) << 17) | ((uint32_t)(FX_ROWS >> 4) << 24);

__device__ __forceinline__ uint32_t x_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t x_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void x_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void x_mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool x_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < FX_WAIT_LIMIT; it++) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok)
                     : "r"(bar), "r"(parity)
                     : "memory");
        if (ok) return true;
        if ((it & 255) == 255 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void x_sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void x_tmem_ld8f(float (&v)[8], uint32_t taddr) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ uint32_t x_h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 x_bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
// low nibbles of bytes 0 and 2 of the word, times the scale: (1024 + w) s - 1024 s, one rounding, exact
__device__ __forceinline__ uint32_t x_scaled_lo(uint32_t word, __half2 s2, __half2 c2) {
    return x_h2_bits(__hfma2(x_bits_h2((word & 0x000f000fu) | 0x64006400u), s2, c2));
}
// high nibbles, left where they are: (1024 + 16 w) (s / 16) - 64 s; s / 16 and 64 s are exact in f16
__device__ __forceinline__ uint32_t x_scaled_hi(uint32_t word, __half2 s16, __half2 c16) {
    return x_h2_bits(__hfma2(x_bits_h2((word & 0x00f000f0u) | 0x64006400u), s16, c16));
}
// an integer 0 .. 1023 in both halves: (1024 + v) - 1024 on the FMA pipe, no integer-to-float conversion
__device__ __forceinline__ __half2 x_small2(uint32_t v) {
    return __hsub2(x_bits_h2(0x64006400u | v | (v << 16)), x_bits_h2(0x64006400u));
}
// signed bytes 0 and 2 of the word (after the sign flip u = y ^ 0x80): (1024 + u) - 1152, exact
__device__ __forceinline__ uint32_t x_signed(uint32_t u, int shift) {
    return x_h2_bits(__hsub2(x_bits_h2(((u >> shift) & 0x00ff00ffu) | 0x64006400u), __float2half2_rn(1152.0f)));
}

struct alignas(16) FxBars {
    uint64_t full[FX_STAGES], empty[FX_STAGES], tfull[FX_TSTAGES], tempty[FX_TSTAGES];
    float da[FX_DA_SLOTS][FX_COLS];
    uint32_t tmem_base;
    int abort_flag;
};

}  // namespace

__global__ void __launch_bounds__(FX_THREADS, 1)
gemm_q4_K_tcgen05_f16x64_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err) {
    extern __shared__ uint8_t fx_raw[];
    __shared__ FxBars bars;
    pdl_trigger();
    const uint32_t smem = (x_smem_u32(fx_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tile0 = (int64_t)blockIdx.y * (FX_ROWS / TILE_ROWS);
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = (int64_t)blockIdx.x * FX_COLS;
    const int64_t K = acts.k;
    const int nh = 2 * nb;   // pipeline steps: half super-blocks
    volatile int *abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < FX_STAGES; i++) {
            x_mbar_init(x_smem_u32(&bars.full[i]), FX_WORK_WARPS);
            x_mbar_init(x_smem_u32(&bars.empty[i]), 1);
        }
        for (int i = 0; i < FX_TSTAGES; i++) {
            x_mbar_init(x_smem_u32(&bars.tfull[i]), 1);
            x_mbar_init(x_smem_u32(&bars.tempty[i]), FX_WORK_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == FX_WORK_WARPS) {
        // all 512 columns: the CTA's shared memory already keeps a second CTA off this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(x_smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;
    pdl_wait();

    if (warp < FX_WORK_WARPS) {
        // ---- conversion share per step: weight piece 4 hs + aj of row (tt, lane); activation piece bk of column bc ----
        const int tt = warp & 3, aj = warp >> 2;
        const bool tile_ok = tile0 + tt < tiles_n;
        const uint8_t *wsrc = tiles + (tile_ok ? tile0 + tt : 0) * (int64_t)nb * 4608 + lane * 16;
        const int prow = tt * 32 + lane;
        // pair within the step gl = aj / 2, 16-byte piece within the pair pp = aj % 2: chunks 8 gl + 4 pp + {0, 1 low | 2, 3 high}
        const uint32_t a_off = (uint32_t)((prow >> 3) * 2048 + (prow & 7) * 16 + (8 * (aj >> 1) + 4 * (aj & 1)) * 128);
        const uint32_t am_off = (uint32_t)(FX_A_BYTES + FX_B_BYTES + (prow >> 3) * 256 + (prow & 7) * 16);
        // column, 16-byte piece of the step's 128 activation bytes: a warp reads 64 contiguous bytes of 8 columns,
        // and each quarter warp stores one 128-byte core-matrix row group
        const int bc = (warp >> 1) * 8 + (lane & 7), bk = 4 * (warp & 1) + (lane >> 3);
        const int64_t bsrc = (col0 + bc < m ? col0 + bc : m - 1) * K + bk * 16;
        // piece bk: pair bk / 4, then (low p0, low p1, high p0, high p1) -> chunks 8 gl + 4 p + 2 hi
        const uint32_t b_off = (uint32_t)(FX_A_BYTES + (bc >> 3) * 2048 + (bc & 7) * 16 + (8 * (bk >> 2) + 4 * (bk & 1) + 2 * ((bk >> 1) & 1)) * 128);
        // sums: lanes 0..7 of every warp, (column, pair of the step); scales: lanes 8..11, one column each
        const bool has_sum = lane < 8, has_da = (lane >> 2) == 2;
        const int sgl = lane & 1, scol_i = warp * 4 + ((lane >> 1) & 3), dcol_i = warp * 4 + (lane & 3);
        const int64_t ssrc = (col0 + scol_i < m ? col0 + scol_i : m - 1) * (K / 16) + 4 * sgl;
        const uint32_t bm_off = (uint32_t)(FX_A_BYTES + FX_B_BYTES + FX_AM_BYTES + sgl * 2048 + (scol_i >> 3) * 256 + (scol_i & 7) * 16);
        const int64_t dsrc = (col0 + dcol_i < m ? col0 + dcol_i : m - 1) * nb;
        // ---- epilogue share: weight row 32 q + lane, activation rows 16 h4 .. + 15 ----
        const int q = warp & 3, h4 = warp >> 2;
        const bool row_ok = tile0 + q < tiles_n;
        const bool any_col = col0 + 16 * h4 < m;
        float sumf[16], summin[16];
#pragma unroll
        for (int c = 0; c < 16; c++) sumf[c] = summin[c] = 0.0f;

        // loads of step 0
        uint4 hd_n = make_uint4(0, 0, 0, 0), w_n = make_uint4(0, 0, 0, 0), y_n;
        short4 bs_n = make_short4(0, 0, 0, 0);
        float dx_n = 0.0f;
        uint32_t dd_cur = 0;   // (d, dmin) of this thread's row: the epilogue row is the conversion row (q = tt)
        if (tile_ok) {
            hd_n = *(const uint4 *)(wsrc);
            w_n = ld_stream16(wsrc + 512 + aj * 512);
        }
        y_n = *(const uint4 *)(acts.qs + bsrc);
        if (has_sum) bs_n = *(const short4 *)(acts.bsums + ssrc);
        if (has_da) dx_n = acts.d[dsrc];

        for (int hb = 0; hb <= nh; hb++) {
            const uint32_t de = dd_cur;   // (d, dmin) of the epilogue row for the super-block of step hb - 1
            if (hb < nh) {
                const int b = hb >> 1, hs = hb & 1;
                const int s = hb % FX_STAGES;
                const uint32_t sph = (uint32_t)(hb / FX_STAGES) & 1u;
                const uint4 hd = hd_n, w = w_n, y = y_n;
                const short4 bs = bs_n;
                const float dx = dx_n;
                dd_cur = hd.x;
                if (!__all_sync(0xffffffffu, x_mbar_wait(x_smem_u32(&bars.empty[s]), sph ^ 1u, abort_flag))) break;
                const uint32_t stage = smem + (uint32_t)(s * FX_STAGE_BYTES);
                if (aj == 0) {
                    const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
                    uint32_t mins[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) mins[j] = x_h2_bits(x_small2(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu));
                    x_sts128(stage + am_off, mins[0], mins[1], mins[2], mins[3]);
                    x_sts128(stage + am_off + 128, mins[4], mins[5], mins[6], mins[7]);
                }
                {
                    // piece c = 4 hs + aj of the row: pair g = c / 2 (sub-blocks 2 g, 2 g + 1)
                    const int g = 2 * hs + (aj >> 1);
                    const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
                    const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
                    const __half2 sl = x_small2(s_lo), sh = x_small2(s_hi);
                    // -1024 s <= 64512 in magnitude: a multiple of 1024 below 65504, exact in f16
                    const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
                    const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
                    const uint32_t x8 = w.x >> 8, y8 = w.y >> 8, z8 = w.z >> 8, w8 = w.w >> 8;   // bytes 1 and 3
                    const uint32_t dstp = stage + a_off;
                    x_sts128(dstp, x_scaled_lo(w.x, sl, cl), x_scaled_lo(x8, sl, cl), x_scaled_lo(w.y, sl, cl), x_scaled_lo(y8, sl, cl));
                    x_sts128(dstp + 128, x_scaled_lo(w.z, sl, cl), x_scaled_lo(z8, sl, cl), x_scaled_lo(w.w, sl, cl), x_scaled_lo(w8, sl, cl));
                    x_sts128(dstp + 256, x_scaled_hi(w.x, sh16, ch), x_scaled_hi(x8, sh16, ch), x_scaled_hi(w.y, sh16, ch), x_scaled_hi(y8, sh16, ch));
                    x_sts128(dstp + 384, x_scaled_hi(w.z, sh16, ch), x_scaled_hi(z8, sh16, ch), x_scaled_hi(w.w, sh16, ch), x_scaled_hi(w8, sh16, ch));
                }
                {
                    const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
                    x_sts128(stage + b_off, x_signed(u0, 0), x_signed(u0, 8), x_signed(u1, 0), x_signed(u1, 8));
                    x_sts128(stage + b_off + 128, x_signed(u2, 0), x_signed(u2, 8), x_signed(u3, 0), x_signed(u3, 8));
                }
                if (has_sum) {
                    // global pair g = 2 hs + sgl: its sums sit in slots 4 g .. 4 g + 3 of the 16
                    const int g = 2 * hs + sgl;
                    const uint32_t xy = x_h2_bits(__halves2half2(__short2half_rn(bs.x), __short2half_rn(bs.y)));
                    const uint32_t zw = x_h2_bits(__halves2half2(__short2half_rn(bs.z), __short2half_rn(bs.w)));
                    const bool odd = g & 1, second = g >> 1;
                    const uint32_t v0 = odd ? 0u : xy, v1 = odd ? 0u : zw, v2 = odd ? xy : 0u, v3 = odd ? zw : 0u;
                    x_sts128(stage + bm_off, second ? 0u : v0, second ? 0u : v1, second ? 0u : v2, second ? 0u : v3);
                    x_sts128(stage + bm_off + 128, second ? v0 : 0u, second ? v1 : 0u, second ? v2 : 0u, second ? v3 : 0u);
                }
                // the activation scales of super-block b, read by every worker while it drains the block's two steps;
                // slot b % 4 is rewritten four super-blocks later, which no worker reaches before all have drained this one
                if (has_da && hs == 0) bars.da[b % FX_DA_SLOTS][dcol_i] = dx;
                // make the stores visible to the tensor core's (async proxy) reads, then hand the stage over
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) x_mbar_arrive(x_smem_u32(&bars.full[s]));
                // the next step's loads, issued once this step's registers are dead; they land while the warp drains
                if (hb + 1 < nh) {
                    const int b1 = (hb + 1) >> 1, hs1 = (hb + 1) & 1;
                    if (tile_ok) {
                        hd_n = *(const uint4 *)(wsrc + (int64_t)b1 * 4608);
                        w_n = ld_stream16(wsrc + (int64_t)b1 * 4608 + 512 + (4 * hs1 + aj) * 512);
                    }
                    y_n = *(const uint4 *)(acts.qs + bsrc + (int64_t)b1 * 256 + hs1 * 128);
                    if (has_sum) bs_n = *(const short4 *)(acts.bsums + ssrc + (int64_t)b1 * 16 + 8 * hs1);
                    if (has_da) dx_n = acts.d[dsrc + b1];
                }
            }
            if (hb >= 1) {
                // ---- drain step e = hb - 1: sumf = fma(f32(ig), d d_x, sumf); summin = fma(f32(mg), dmin d_x, summin) ----
                const int e = hb - 1, t = e % FX_TSTAGES, be = e >> 1;
                const uint32_t tph = (uint32_t)(e / FX_TSTAGES) & 1u;
                // full[] of that step completed long ago; waiting on it orders this warp's reads of da[] after the store
                const bool ready = x_mbar_wait(x_smem_u32(&bars.full[e % FX_STAGES]), (uint32_t)(e / FX_STAGES) & 1u, abort_flag) &&
                                   x_mbar_wait(x_smem_u32(&bars.tfull[t]), tph, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float dw = f16_bits_to_f32((uint16_t)(de & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(de >> 16));
                const float4 *das = reinterpret_cast<const float4 *>(bars.da[be % FX_DA_SLOTS] + 16 * h4);
                const uint32_t trow = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(t * 256 + 16 * h4);
#pragma unroll
                for (int pc = 0; pc < 4; pc++) {
                    const int gl = pc >> 1, c0 = 8 * (pc & 1);
                    float ig[8], mg[8];
                    x_tmem_ld8f(ig, trow + (uint32_t)(gl * FX_COLS + c0));
                    x_tmem_ld8f(mg, trow + (uint32_t)(128 + gl * FX_COLS + c0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (pc == 3) {
                        // the accumulator stage is free again once every worker warp has read it
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) x_mbar_arrive(x_smem_u32(&bars.tempty[t]));
                    }
                    if (any_col) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const float4 dq = das[c0 / 4 + h];
                            const float dxs[4] = {dq.x, dq.y, dq.z, dq.w};
#pragma unroll
                            for (int c4 = 0; c4 < 4; c4++) {
                                const int c = 4 * h + c4;
                                sumf[c0 + c] = __fmaf_rn(ig[c], __fmul_rn(dw, dxs[c4]), sumf[c0 + c]);
                                summin[c0 + c] = __fmaf_rn(mg[c], __fmul_rn(dmw, dxs[c4]), summin[c0 + c]);
                            }
                        }
                    }
                }
            }
        }
        const int64_t row = (tile0 + q) * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 16; c++) {
                const int64_t col = col0 + 16 * h4 + c;
                if (col < m) dst[col * lddst + row] = __fsub_rn(sumf[c], summin[c]);
            }
        }
    }
    else if (lane == 0) {
        // ---- MMA issue: per step two pairs x (four K = 16 MMAs for ig, one for mg) ----
        for (int hb = 0; hb < nh; hb++) {
            const int s = hb % FX_STAGES, t = hb % FX_TSTAGES;
            const uint32_t sph = (uint32_t)(hb / FX_STAGES) & 1u, tph = (uint32_t)(hb / FX_TSTAGES) & 1u;
            if (!x_mbar_wait(x_smem_u32(&bars.full[s]), sph, abort_flag)) break;
            if (!x_mbar_wait(x_smem_u32(&bars.tempty[t]), tph ^ 1u, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = smem + (uint32_t)(s * FX_STAGE_BYTES), b_base = a_base + FX_A_BYTES;
            const uint32_t am_base = b_base + FX_B_BYTES, bm_base = am_base + FX_AM_BYTES;
#pragma unroll
            for (int gl = 0; gl < 2; gl++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint64_t adesc = x_desc(a_base + (8 * gl + 2 * i) * 128, 128, 2048);
                    const uint64_t bdesc = x_desc(b_base + (8 * gl + 2 * i) * 128, 128, 2048);
                    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(
                                     tmem + (uint32_t)(t * 256 + gl * FX_COLS)),
                                 "l"(adesc), "l"(bdesc), "r"(FX_IDESC), "r"(i)
                                 : "memory");
                }
                const uint64_t amdesc = x_desc(am_base, 128, 256), bmdesc = x_desc(bm_base + gl * 2048, 128, 256);
                asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(
                                 tmem + (uint32_t)(t * 256 + 128 + gl * FX_COLS)),
                             "l"(amdesc), "l"(bmdesc), "r"(FX_IDESC), "r"(0)
                             : "memory");
            }
            // both arrive when the MMAs above have completed: operands consumed, accumulators ready
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(x_smem_u32(&bars.empty[s])) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(x_smem_u32(&bars.tfull[t])) : "memory");
        }
    }
    // ---- teardown: every role has left its loop (finished, or gave up) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FX_WORK_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, FX_ERR_WAIT);
}

int launch_gemm_tcgen05_f16x64(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_f16x64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FX_SMEM_BYTES));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const int nb = (int)(k / GROUP_K);
    const int64_t gx = (m + FX_COLS - 1) / FX_COLS, gy = (n + FX_ROWS - 1) / FX_ROWS;
    B200_REQUIRE(gx < 0x7fffffffLL && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    return launch_pdl(gemm_q4_K_tcgen05_f16x64_kernel, dim3((unsigned)gx, (unsigned)gy), dim3(FX_THREADS), (size_t)FX_SMEM_BYTES, s, tiles, acts,
                      dst, lddst, n, nb, m, err);
}

}  // namespace b200
