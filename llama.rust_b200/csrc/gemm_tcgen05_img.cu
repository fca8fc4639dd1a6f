// Q4_K prompt mat-mul, 8x8 gemm chain, in two passes: the operands are first expanded to f16 in exactly the
// shared-memory images the tensor core reads, then a mat-mul kernel that does no conversion at all moves
// those images with bulk copies and spends its warps on the chain's epilogue.
//
// Why: in the one-pass kernels (gemm_tcgen05.cu, gemm_tcgen05_f16.cu) every CTA converts its own operands, so
// the weights of a 128-row block are converted once per 64 activation rows and the activations once per 128
// weight rows, and conversion (loads, nibble arithmetic, 57 KB of shared-memory stores per step) and the
// accumulator drain take turns on the same warps: measured, 2300 + 1900 cycles per step against 1280 cycles of
// tensor-core work.  Expanding once per mat-mul costs 2.25 bytes written per weight (read back through L2 by the
// CTAs of a row block, which run side by side) and removes the conversion from the inner loop.
//
// Arithmetic (gemm_tcgen05.cu has the argument): per sub-block pair g the chain needs the integers
//     ig = s_lo dot_lo + s_hi dot_hi  (< 2^23)      mg = m_lo bsum_lo + m_hi bsum_hi  (< 2^19)
// as f32.  s * w (<= 945), the activation bytes, the mins and the 16-element activation sums (<= 2032) are exact
// in f16 and every partial sum is an integer below 2^24, so an f16 x f16 -> f32 MMA returns exactly f32(ig) and
// f32(mg); the epilogue is the chain's own two fused multiply-adds per pair,
//     sumf = fma(f32(ig), d d_x, sumf);  summin = fma(f32(mg), dmin d_x, summin);  out = sumf - summin
// (crates/ggml/src/repack.rs:1692-1768).
//
// Images, one per pipeline step (half a super-block = two sub-block pairs), K-major, no swizzle, 8 rows x 16
// bytes core matrices with K-adjacent ones 128 bytes apart:
//   weights     [128-row block][step]  A  [128 rows][128 f16]  s * w, K order within a pair: 16-byte piece p,
//                                          (low | high) nibbles, bytes (0,2,1,3 ..)                  32768 B
//                                      Am [128 rows][16 f16]  slots 4g, 4g+1 = m_lo of pair g, 4g+2, 4g+3 = m_hi  4096 B
//   activations [64-row block][step]   B  [64 rows][128 f16]  the bytes in the same K order              16384 B
//                                      Bm [2 pairs][64 rows][16 f16]  slots 4g .. 4g+3 = the pair's four sums, rest 0  4096 B
//               [64-row block][super-block]  64 f32 activation scales d_x                                    256 B
// Every wait is bounded; a wait that runs out raises the CTA's abort flag and the device error word.
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int IM_ROWS = 128, IM_COLS = 64;
constexpr int IM_EPI_WARPS = 16, IM_MMA_WARP = 16, IM_LOAD_WARP = 17;
constexpr int IM_THREADS = 20 * 32;   // four epilogue warp groups + one for the two single-thread roles (two warps idle)
constexpr int IM_REGS_EPI = 112, IM_REGS_CTL = 32;   // 512 x 112 + 128 x 32 = 640 x 96, what the CTA is launched with
constexpr int IM_EXPAND_THREADS = 512;
constexpr int IM_STAGES = 3, IM_TSTAGES = 2;
constexpr int IM_A_BYTES = IM_ROWS * 256, IM_AM_BYTES = IM_ROWS * 32;
constexpr int IM_B_BYTES = IM_COLS * 256, IM_BM_BYTES = 2 * IM_COLS * 32;
constexpr int IM_AIMG = IM_A_BYTES + IM_AM_BYTES;   // 36864
constexpr int IM_BIMG = IM_B_BYTES + IM_BM_BYTES;   // 20480
constexpr int IM_STAGE_BYTES = IM_AIMG + IM_BIMG;   // 57344
constexpr int IM_SMEM_BYTES = IM_STAGES * IM_STAGE_BYTES + 1024;
constexpr int IM_DA_SLOTS = 4, IM_DA_BYTES = IM_COLS * 4;
constexpr uint32_t IM_WAIT_LIMIT = 1u << 22;
constexpr int IM_ERR_WAIT = 4;
// kind::f16 instruction descriptor: f32 accumulator, f16 x f16, both operands K-major, N = 64, M = 128
constexpr uint32_t IM_IDESC = (1u << 4) | ((uint32_t)(IM_COLS >> 3) << 17) | ((uint32_t)(IM_ROWS >> 4) << 24);

__device__ __forceinline__ uint32_t i_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t i_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void i_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void i_mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void i_mbar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy, one destination CTA; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void i_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool i_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < IM_WAIT_LIMIT; it++) {
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
__device__ __forceinline__ void i_tmem_ld8f(float (&v)[8], uint32_t taddr) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ uint32_t i_h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 i_bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
// low nibbles of bytes 0 and 2 of the word, times the scale: (1024 + w) s - 1024 s, one rounding, exact
__device__ __forceinline__ uint32_t i_scaled_lo(uint32_t word, __half2 s2, __half2 c2) {
    return i_h2_bits(__hfma2(i_bits_h2((word & 0x000f000fu) | 0x64006400u), s2, c2));
}
// high nibbles, left where they are: (1024 + 16 w) (s / 16) - 64 s; s / 16 and 64 s are exact in f16
__device__ __forceinline__ uint32_t i_scaled_hi(uint32_t word, __half2 s16, __half2 c16) {
    return i_h2_bits(__hfma2(i_bits_h2((word & 0x00f000f0u) | 0x64006400u), s16, c16));
}
// an integer 0 .. 1023 in both halves: (1024 + v) - 1024
__device__ __forceinline__ __half2 i_small2(uint32_t v) { return __hsub2(i_bits_h2(0x64006400u | v | (v << 16)), i_bits_h2(0x64006400u)); }
// signed bytes 0 and 2 of the word (after the sign flip u = y ^ 0x80): (1024 + u) - 1152, exact
__device__ __forceinline__ uint32_t i_signed(uint32_t u, int shift) {
    return i_h2_bits(__hsub2(i_bits_h2(((u >> shift) & 0x00ff00ffu) | 0x64006400u), __float2half2_rn(1152.0f)));
}
__device__ __forceinline__ void i_stg128(uint8_t *p, uint32_t x, uint32_t y, uint32_t z, uint32_t w) { *reinterpret_cast<uint4 *>(p) = make_uint4(x, y, z, w); }

// All MMAs of one 64-column step in one statement, so that the issuing thread spends three instructions per MMA
// (two descriptor adds and the MMA) instead of rebuilding descriptors and predicates each time.  Descriptor start
// addresses count 16-byte units: K step i is + 16 (two 128-byte core-matrix columns), pair gl + 64; Bm of pair gl
// + 128 (2048 bytes).  d0 = the tensor-memory stage: ig of pair gl at + 64 gl, mg at + 128 + 64 gl.
__device__ __forceinline__ void i_issue_step64(uint32_t d0, uint64_t adesc0, uint64_t bdesc0, uint64_t amdesc, uint64_t bmdesc0, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred pn, py;\n"
        ".reg .b64 a, b;\n"
        ".reg .b32 d;\n"
        "setp.ne.b32 pn, 0, 0;\n"
        "setp.eq.b32 py, 0, 0;\n"
        // pair 0
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %5, pn;\n"
        "add.u64 a, %1, 16;  add.u64 b, %2, 16;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u64 a, %1, 32;  add.u64 b, %2, 32;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u64 a, %1, 48;  add.u64 b, %2, 48;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u32 d, %0, 128;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], %3, %4, %5, pn;\n"
        // pair 1
        "add.u32 d, %0, 64;\n"
        "add.u64 a, %1, 64;  add.u64 b, %2, 64;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], a, b, %5, pn;\n"
        "add.u64 a, %1, 80;  add.u64 b, %2, 80;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], a, b, %5, py;\n"
        "add.u64 a, %1, 96;  add.u64 b, %2, 96;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], a, b, %5, py;\n"
        "add.u64 a, %1, 112; add.u64 b, %2, 112;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], a, b, %5, py;\n"
        "add.u32 d, %0, 192;\n"
        "add.u64 b, %4, 128;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], %3, b, %5, pn;\n"
        "}\n" ::"r"(d0),
        "l"(adesc0), "l"(bdesc0), "l"(amdesc), "l"(bmdesc0), "r"(idesc)
        : "memory");
}
// The five MMAs of one 128-column step (one pair): ig at d0, mg at d0 + 128.
__device__ __forceinline__ void i_issue_step128(uint32_t d0, uint64_t adesc0, uint64_t bdesc0, uint64_t amdesc, uint64_t bmdesc, uint32_t idesc) {
    asm volatile(
        "{\n"
        ".reg .pred pn, py;\n"
        ".reg .b64 a, b;\n"
        ".reg .b32 d;\n"
        "setp.ne.b32 pn, 0, 0;\n"
        "setp.eq.b32 py, 0, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %5, pn;\n"
        "add.u64 a, %1, 16;  add.u64 b, %2, 16;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u64 a, %1, 32;  add.u64 b, %2, 32;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u64 a, %1, 48;  add.u64 b, %2, 48;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %5, py;\n"
        "add.u32 d, %0, 128;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [d], %3, %4, %5, pn;\n"
        "}\n" ::"r"(d0),
        "l"(adesc0), "l"(bdesc0), "l"(amdesc), "l"(bmdesc), "r"(idesc)
        : "memory");
}

struct alignas(16) ImBars {
    uint64_t full[IM_STAGES], empty[IM_STAGES], tfull[IM_TSTAGES], tempty[IM_TSTAGES];
    float da[IM_DA_SLOTS][IM_COLS];
    uint32_t tmem_base;
    int abort_flag;
};

}  // namespace

// Weights of one 128-row block and one super-block -> the A / Am images of its two steps.  Warp (tt, aj): row
// (tile tt, lane), 16-byte piece 4 hs + aj of the row's 128 nibble bytes.
__global__ void __launch_bounds__(IM_EXPAND_THREADS) expand_q4_K_weights_kernel(const uint8_t *__restrict__ tiles, uint8_t *aimg, int64_t tiles_n, int nb) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tt = warp & 3, aj = warp >> 2;
    const int b = blockIdx.x;
    const int64_t rb = blockIdx.y, tile = rb * 4 + tt;
    const bool tile_ok = tile < tiles_n;
    const uint8_t *src = tiles + ((tile_ok ? tile : 0) * (int64_t)nb + b) * 4608 + lane * 16;
    uint4 hd = make_uint4(0, 0, 0, 0), wq[2] = {hd, hd};
    if (tile_ok) {
        // the weights do not depend on the previous kernel
        hd = *(const uint4 *)(src);
        wq[0] = ld_stream16(src + 512 + aj * 512);
        wq[1] = ld_stream16(src + 512 + (4 + aj) * 512);
    }
    pdl_wait();   // the previous mat-mul may still be reading the images
    const int prow = tt * 32 + lane;
    // pair within the step gl = aj / 2, piece within the pair pp = aj % 2: chunks 8 gl + 4 pp + {0, 1 low | 2, 3 high}
    const int a_off = (prow >> 3) * 2048 + (prow & 7) * 16 + (8 * (aj >> 1) + 4 * (aj & 1)) * 128;
    const int am_off = IM_A_BYTES + (prow >> 3) * 256 + (prow & 7) * 16;
#pragma unroll
    for (int hs = 0; hs < 2; hs++) {
        uint8_t *img = aimg + (rb * 2 * nb + 2 * b + hs) * (int64_t)IM_AIMG;
        const uint4 w = wq[hs];
        if (aj == 0) {
            const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
            uint32_t mins[8];
#pragma unroll
            for (int j = 0; j < 8; j++) mins[j] = i_h2_bits(i_small2(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu));
            i_stg128(img + am_off, mins[0], mins[1], mins[2], mins[3]);
            i_stg128(img + am_off + 128, mins[4], mins[5], mins[6], mins[7]);
        }
        // piece c = 4 hs + aj of the row: pair g = c / 2 (sub-blocks 2 g, 2 g + 1)
        const int g = 2 * hs + (aj >> 1);
        const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
        const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
        const __half2 sl = i_small2(s_lo), sh = i_small2(s_hi);
        // -1024 s <= 64512 in magnitude: a multiple of 1024 below 65504, exact in f16
        const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
        const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
        const uint32_t x8 = w.x >> 8, y8 = w.y >> 8, z8 = w.z >> 8, w8 = w.w >> 8;   // bytes 1 and 3
        uint8_t *dstp = img + a_off;
        i_stg128(dstp, i_scaled_lo(w.x, sl, cl), i_scaled_lo(x8, sl, cl), i_scaled_lo(w.y, sl, cl), i_scaled_lo(y8, sl, cl));
        i_stg128(dstp + 128, i_scaled_lo(w.z, sl, cl), i_scaled_lo(z8, sl, cl), i_scaled_lo(w.w, sl, cl), i_scaled_lo(w8, sl, cl));
        i_stg128(dstp + 256, i_scaled_hi(w.x, sh16, ch), i_scaled_hi(x8, sh16, ch), i_scaled_hi(w.y, sh16, ch), i_scaled_hi(y8, sh16, ch));
        i_stg128(dstp + 384, i_scaled_hi(w.z, sh16, ch), i_scaled_hi(z8, sh16, ch), i_scaled_hi(w.w, sh16, ch), i_scaled_hi(w8, sh16, ch));
    }
}

// Q8_K activations of one 64-row block and one super-block -> the B / Bm images of its two steps and the scales.
__global__ void __launch_bounds__(IM_EXPAND_THREADS) expand_q8_K_acts_kernel(ActView acts, uint8_t *bimg, float *daimg, int64_t m, int nb) {
    pdl_trigger();
    pdl_wait();   // the activations come from the previous kernel
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x;
    const int64_t cb = blockIdx.y, K = acts.k;
    // a warp reads 64 contiguous bytes of 8 activation rows; each quarter warp writes one 128-byte row group
    const int bc = (warp >> 1) * 8 + (lane & 7), bk = 4 * (warp & 1) + (lane >> 3);
    const int64_t col = cb * IM_COLS + bc;
    // piece bk: pair bk / 4, then (low p0, low p1, high p0, high p1) -> chunks 8 gl + 4 p + 2 hi
    const int b_off = (bc >> 3) * 2048 + (bc & 7) * 16 + (8 * (bk >> 2) + 4 * (bk & 1) + 2 * ((bk >> 1) & 1)) * 128;
    // sums: lanes 0..7 of every warp, (row, pair of the step); scales: lanes 8..11, one row each
    const bool has_sum = lane < 8, has_da = (lane >> 2) == 2;
    const int sgl = lane & 1, scol_i = warp * 4 + ((lane >> 1) & 3), dcol_i = warp * 4 + (lane & 3);
    const int64_t scol = cb * IM_COLS + scol_i, dcol = cb * IM_COLS + dcol_i;
    const int bm_off = IM_B_BYTES + sgl * 2048 + (scol_i >> 3) * 256 + (scol_i & 7) * 16;
#pragma unroll
    for (int hs = 0; hs < 2; hs++) {
        uint8_t *img = bimg + (cb * 2 * nb + 2 * b + hs) * (int64_t)IM_BIMG;
        uint4 y = make_uint4(0, 0, 0, 0);
        if (col < m) y = *(const uint4 *)(acts.qs + col * K + (int64_t)b * 256 + hs * 128 + bk * 16);
        const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
        i_stg128(img + b_off, i_signed(u0, 0), i_signed(u0, 8), i_signed(u1, 0), i_signed(u1, 8));
        i_stg128(img + b_off + 128, i_signed(u2, 0), i_signed(u2, 8), i_signed(u3, 0), i_signed(u3, 8));
        if (has_sum) {
            short4 bs = make_short4(0, 0, 0, 0);
            if (scol < m) bs = *(const short4 *)(acts.bsums + scol * (K / 16) + (int64_t)b * 16 + 8 * hs + 4 * sgl);
            // global pair g = 2 hs + sgl: its sums sit in slots 4 g .. 4 g + 3 of the 16
            const int g = 2 * hs + sgl;
            const uint32_t xy = i_h2_bits(__halves2half2(__short2half_rn(bs.x), __short2half_rn(bs.y)));
            const uint32_t zw = i_h2_bits(__halves2half2(__short2half_rn(bs.z), __short2half_rn(bs.w)));
            const bool odd = g & 1, second = g >> 1;
            const uint32_t v0 = odd ? 0u : xy, v1 = odd ? 0u : zw, v2 = odd ? xy : 0u, v3 = odd ? zw : 0u;
            i_stg128(img + bm_off, second ? 0u : v0, second ? 0u : v1, second ? 0u : v2, second ? 0u : v3);
            i_stg128(img + bm_off + 128, second ? v0 : 0u, second ? v1 : 0u, second ? v2 : 0u, second ? v3 : 0u);
        }
    }
    if (has_da) daimg[(cb * nb + b) * IM_COLS + dcol_i] = dcol < m ? acts.d[dcol * nb + b] : 0.0f;
}

// 128 x 64 outputs per CTA.  Warp 17 (one thread) copies each step's images into a three-stage ring, warp 16 (one
// thread) issues the step's MMAs into one of two tensor-memory stages (2 pairs x (ig, mg) x 64 columns each),
// warps 0..15 drain: warp w owns rows 32 (w % 4) .. + 31 (its tensor-memory lanes) and columns 16 (w / 4) .. + 15.
__global__ void __launch_bounds__(IM_THREADS, 1)
gemm_q4_K_tcgen05_img_kernel(const uint8_t *__restrict__ tiles, const uint8_t *__restrict__ aimg, const uint8_t *__restrict__ bimg,
                             const float *__restrict__ daimg, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err) {
    extern __shared__ uint8_t im_raw[];
    __shared__ ImBars bars;
    pdl_trigger();
    const uint32_t smem = (i_smem_u32(im_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t rb = blockIdx.y, cb = blockIdx.x;
    const int64_t tile0 = rb * (IM_ROWS / TILE_ROWS), tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = cb * IM_COLS;
    const int nh = 2 * nb;   // pipeline steps: half super-blocks
    volatile int *abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < IM_STAGES; i++) {
            i_mbar_init(i_smem_u32(&bars.full[i]), 1);    // the loader's arrive + the bytes it announced
            i_mbar_init(i_smem_u32(&bars.empty[i]), 1);   // the MMA thread's commit
        }
        for (int i = 0; i < IM_TSTAGES; i++) {
            i_mbar_init(i_smem_u32(&bars.tfull[i]), 1);
            i_mbar_init(i_smem_u32(&bars.tempty[i]), IM_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == IM_MMA_WARP) {
        // all 512 columns: the CTA's shared memory already keeps a second CTA off this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(i_smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;
    // A CTA of 20 warps starts with 96 registers per thread (five warps share a scheduler's 16384).  The control
    // warp group gives 64 of them back and the epilogue warp groups take 16 more each: the pool balances exactly.
    if (warp < IM_EPI_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(IM_REGS_EPI));
        pdl_wait();   // the images are the two previous kernels' output
        const int q = warp & 3, h4 = warp >> 2;
        const bool row_ok = tile0 + q < tiles_n;
        const bool any_col = col0 + 16 * h4 < m;
        // (d, dmin) of this thread's row, one word per super-block, fetched one super-block ahead
        const uint8_t *hdr = tiles + (row_ok ? tile0 + q : 0) * (int64_t)nb * 4608 + lane * 16;
        uint32_t dd_next = row_ok ? *(const uint32_t *)(hdr) : 0u;
        float dw = 0.0f, dmw = 0.0f;
        float sumf[16], summin[16];
#pragma unroll
        for (int c = 0; c < 16; c++) sumf[c] = summin[c] = 0.0f;
        const uint32_t trow0 = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(16 * h4);

        for (int e = 0; e < nh; e++) {
            const int t = e % IM_TSTAGES, be = e >> 1;
            if ((e & 1) == 0) {
                dw = f16_bits_to_f32((uint16_t)(dd_next & 0xffffu));
                dmw = f16_bits_to_f32((uint16_t)(dd_next >> 16));
                if (be + 1 < nb && row_ok) dd_next = *(const uint32_t *)(hdr + (int64_t)(be + 1) * 4608);
            }
            // the accumulators of step e are complete; so are the copies the MMAs waited for, the scales among them
            if (!__all_sync(0xffffffffu, i_mbar_wait(i_smem_u32(&bars.tfull[t]), (uint32_t)(e / IM_TSTAGES) & 1u, abort_flag))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float4 *das = reinterpret_cast<const float4 *>(bars.da[be % IM_DA_SLOTS] + 16 * h4);
            const uint32_t trow = trow0 + (uint32_t)(t * 256);
            // four rounds r = (columns c0 = 8 (r / 2) .. + 7, pair gl = r % 2): sumf = fma(f32(ig), d d_x, sumf);
            // summin = fma(f32(mg), dmin d_x, summin).  Three rounds' loads go out together, the fourth reuses the
            // first one's registers and lands while rounds 1 and 2 are computed; the two pairs of a column group
            // follow each other so that the products d d_x, dmin d_x are made once per group.
            float ig[3][8], mg[3][8], pd[8], pm[8];
#pragma unroll
            for (int r = 0; r < 3; r++) {
                i_tmem_ld8f(ig[r], trow + (uint32_t)((r & 1) * IM_COLS + 8 * (r >> 1)));
                i_tmem_ld8f(mg[r], trow + (uint32_t)(128 + (r & 1) * IM_COLS + 8 * (r >> 1)));
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int c0 = 8 * (r >> 1), buf = r == 3 ? 0 : r;
                if (r == 3) {
                    // every value of the stage is in registers: hand it back to the MMA thread
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) i_mbar_arrive(i_smem_u32(&bars.tempty[t]));
                }
                if (any_col) {
                    if ((r & 1) == 0) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const float4 dq = das[c0 / 4 + h];
                            const float dxs[4] = {dq.x, dq.y, dq.z, dq.w};
#pragma unroll
                            for (int c4 = 0; c4 < 4; c4++) {
                                pd[4 * h + c4] = __fmul_rn(dw, dxs[c4]);
                                pm[4 * h + c4] = __fmul_rn(dmw, dxs[c4]);
                            }
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        sumf[c0 + c] = __fmaf_rn(ig[buf][c], pd[c], sumf[c0 + c]);
                        summin[c0 + c] = __fmaf_rn(mg[buf][c], pm[c], summin[c0 + c]);
                    }
                }
                if (r == 0) {
                    // the fourth group of loads goes into the first group's registers, now consumed
                    i_tmem_ld8f(ig[0], trow + (uint32_t)(IM_COLS + 8));
                    i_tmem_ld8f(mg[0], trow + (uint32_t)(128 + IM_COLS + 8));
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
    } else {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(IM_REGS_CTL));
      pdl_wait();
      if (warp == IM_MMA_WARP) {
        if (lane == 0) {
            // per step: two pairs x (four K = 16 MMAs for ig, one for mg)
            for (int hb = 0; hb < nh; hb++) {
                const int s = hb % IM_STAGES, t = hb % IM_TSTAGES;
                if (!i_mbar_wait(i_smem_u32(&bars.full[s]), (uint32_t)(hb / IM_STAGES) & 1u, abort_flag)) break;
                if (!i_mbar_wait(i_smem_u32(&bars.tempty[t]), ((uint32_t)(hb / IM_TSTAGES) & 1u) ^ 1u, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_base = smem + (uint32_t)(s * IM_STAGE_BYTES), am_base = a_base + IM_A_BYTES;
                const uint32_t b_base = a_base + IM_AIMG, bm_base = b_base + IM_B_BYTES;
                // Am holds the mins of all four pairs, Bm is zero outside the slots of global pair 2 hs + gl
                i_issue_step64(tmem + (uint32_t)(t * 256), i_desc(a_base, 128, 2048), i_desc(b_base, 128, 2048), i_desc(am_base, 128, 256),
                               i_desc(bm_base, 128, 256), IM_IDESC);
                // both arrive when the MMAs above have completed: images consumed, accumulators ready
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(i_smem_u32(&bars.empty[s])) : "memory");
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(i_smem_u32(&bars.tfull[t])) : "memory");
            }
        }
      } else if (warp == IM_LOAD_WARP && lane == 0) {
        // ---- loader: the images of step hb into stage hb % 3, the scales of a super-block with its first step ----
        const uint8_t *asrc = aimg + rb * nh * (int64_t)IM_AIMG, *bsrc = bimg + cb * nh * (int64_t)IM_BIMG;
        const float *dsrc = daimg + cb * nb * (int64_t)IM_COLS;
        int issued = -1;
        for (int hb = 0; hb < nh; hb++) {
            const int s = hb % IM_STAGES;
            if (!i_mbar_wait(i_smem_u32(&bars.empty[s]), ((uint32_t)(hb / IM_STAGES) & 1u) ^ 1u, abort_flag)) break;
            const uint32_t bar = i_smem_u32(&bars.full[s]), stage = smem + (uint32_t)(s * IM_STAGE_BYTES);
            const bool first = (hb & 1) == 0;
            i_mbar_expect(bar, (uint32_t)(IM_STAGE_BYTES + (first ? IM_DA_BYTES : 0)));
            i_bulk_load(stage, asrc + (int64_t)hb * IM_AIMG, IM_AIMG, bar);
            i_bulk_load(stage + IM_AIMG, bsrc + (int64_t)hb * IM_BIMG, IM_BIMG, bar);
            // slot b % 4 is rewritten four super-blocks later: the stage this step reuses was released by MMAs
            // that had waited for the drain of every step of that older super-block
            if (first) i_bulk_load(i_smem_u32(bars.da[(hb >> 1) % IM_DA_SLOTS]), dsrc + (int64_t)(hb >> 1) * IM_COLS, IM_DA_BYTES, bar);
            issued = hb;
        }
        // gave up somewhere: let the copies already in flight land before the CTA's shared memory goes away
        if (*abort_flag && issued >= 0) i_mbar_wait(i_smem_u32(&bars.full[issued % IM_STAGES]), (uint32_t)(issued / IM_STAGES) & 1u, abort_flag);
      }
    }
    // ---- teardown: every role has left its loop (finished, or gave up) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == IM_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, IM_ERR_WAIT);
}

// ---- 128 activation rows per CTA, one sub-block pair per step ------------------------------------------------
// The 64-column kernel above is bound by shared-memory bandwidth: each of a step's 18 MMAs re-reads its 4 KB of A
// for 64 columns while the bulk copies write the next images (164 KB through a 128 B/cycle port per step).  With
// N = 128 an MMA's A read serves twice the columns.  Tensor memory holds two stages of (ig, mg) x 128 columns only
// if a step is one pair, so the images are cut per pair: A [128 rows][64 f16] 16 KB + Am 4 KB, B [128 rows][64 f16]
// 16 KB + Bm [128 rows][16 f16] 4 KB, five 40 KB stages.
namespace {
constexpr int IW_COLS = 128;
constexpr int IW_STAGES = 5;
constexpr int IW_A_BYTES = IM_ROWS * 128, IW_AM_BYTES = IM_ROWS * 32;
constexpr int IW_B_BYTES = IW_COLS * 128, IW_BM_BYTES = IW_COLS * 32;
constexpr int IW_AIMG = IW_A_BYTES + IW_AM_BYTES;   // 20480
constexpr int IW_BIMG = IW_B_BYTES + IW_BM_BYTES;   // 20480
constexpr int IW_STAGE_BYTES = IW_AIMG + IW_BIMG;   // 40960
constexpr int IW_SMEM_BYTES = IW_STAGES * IW_STAGE_BYTES + 1024;
constexpr int IW_DA_BYTES = IW_COLS * 4;
constexpr uint32_t IW_IDESC = (1u << 4) | ((uint32_t)(IW_COLS >> 3) << 17) | ((uint32_t)(IM_ROWS >> 4) << 24);
struct alignas(16) IwBars {
    uint64_t full[IW_STAGES], empty[IW_STAGES], tfull[IM_TSTAGES], tempty[IM_TSTAGES];
    float da[IM_DA_SLOTS][IW_COLS];
    uint32_t tmem_base;
    int abort_flag;
};
}  // namespace

// Weights of one 128-row block and one super-block -> the A / Am images of its four steps.  Warp (tt, aj): row
// (tile tt, lane), 16-byte pieces aj and 4 + aj of the row's 128 nibble bytes, and the Am image of step aj.
__global__ void __launch_bounds__(IM_EXPAND_THREADS) expand_q4_K_weights_pair_kernel(const uint8_t *__restrict__ tiles, uint8_t *aimg, int64_t tiles_n, int nb) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tt = warp & 3, aj = warp >> 2;
    const int b = blockIdx.x;
    const int64_t rb = blockIdx.y, tile = rb * 4 + tt;
    const bool tile_ok = tile < tiles_n;
    const uint8_t *src = tiles + ((tile_ok ? tile : 0) * (int64_t)nb + b) * 4608 + lane * 16;
    uint4 hd = make_uint4(0, 0, 0, 0), wq[2] = {hd, hd};
    if (tile_ok) {
        hd = *(const uint4 *)(src);
        wq[0] = ld_stream16(src + 512 + aj * 512);
        wq[1] = ld_stream16(src + 512 + (4 + aj) * 512);
    }
    pdl_wait();   // the previous mat-mul may still be reading the images
    const int prow = tt * 32 + lane;
    uint8_t *img0 = aimg + (rb * 4 * nb + 4 * b) * (int64_t)IW_AIMG;
    {
        // all eight mins into the Am image of step aj (Bm selects the pair)
        const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
        uint32_t mins[8];
#pragma unroll
        for (int j = 0; j < 8; j++) mins[j] = i_h2_bits(i_small2(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu));
        uint8_t *am = img0 + aj * (int64_t)IW_AIMG + IW_A_BYTES + (prow >> 3) * 256 + (prow & 7) * 16;
        i_stg128(am, mins[0], mins[1], mins[2], mins[3]);
        i_stg128(am + 128, mins[4], mins[5], mins[6], mins[7]);
    }
    // piece within the pair pp = aj % 2: chunks 4 pp + {0, 1 low | 2, 3 high}
    const int a_off = (prow >> 3) * 1024 + (prow & 7) * 16 + 4 * (aj & 1) * 128;
#pragma unroll
    for (int hs = 0; hs < 2; hs++) {
        // piece c = 4 hs + aj of the row: pair g = c / 2 (sub-blocks 2 g, 2 g + 1)
        const int g = 2 * hs + (aj >> 1);
        const uint4 w = wq[hs];
        const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
        const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
        const __half2 sl = i_small2(s_lo), sh = i_small2(s_hi);
        const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
        const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
        const uint32_t x8 = w.x >> 8, y8 = w.y >> 8, z8 = w.z >> 8, w8 = w.w >> 8;   // bytes 1 and 3
        uint8_t *dstp = img0 + g * (int64_t)IW_AIMG + a_off;
        i_stg128(dstp, i_scaled_lo(w.x, sl, cl), i_scaled_lo(x8, sl, cl), i_scaled_lo(w.y, sl, cl), i_scaled_lo(y8, sl, cl));
        i_stg128(dstp + 128, i_scaled_lo(w.z, sl, cl), i_scaled_lo(z8, sl, cl), i_scaled_lo(w.w, sl, cl), i_scaled_lo(w8, sl, cl));
        i_stg128(dstp + 256, i_scaled_hi(w.x, sh16, ch), i_scaled_hi(x8, sh16, ch), i_scaled_hi(w.y, sh16, ch), i_scaled_hi(y8, sh16, ch));
        i_stg128(dstp + 384, i_scaled_hi(w.z, sh16, ch), i_scaled_hi(z8, sh16, ch), i_scaled_hi(w.w, sh16, ch), i_scaled_hi(w8, sh16, ch));
    }
}

// Q8_K activations of one 128-row block and one super-block -> the B / Bm images of its four steps and the scales.
__global__ void __launch_bounds__(IM_EXPAND_THREADS) expand_q8_K_acts_pair_kernel(ActView acts, uint8_t *bimg, float *daimg, int64_t m, int nb) {
    pdl_trigger();
    pdl_wait();   // the activations come from the previous kernel
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int b = blockIdx.x;
    const int64_t cb = blockIdx.y, K = acts.k;
    uint8_t *img0 = bimg + (cb * 4 * nb + 4 * b) * (int64_t)IW_BIMG;
    // a warp reads 64 contiguous bytes (one pair) of 8 activation rows; each quarter warp writes one 128-byte row group
    const int bc = warp * 8 + (lane & 7), r = lane >> 3;
    const int64_t col = cb * IW_COLS + bc;
    // piece r of the pair: (low p0, low p1, high p0, high p1) -> chunks 4 p + 2 hi
    const int b_off = (bc >> 3) * 1024 + (bc & 7) * 16 + (4 * (r & 1) + 2 * (r >> 1)) * 128;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint4 y = make_uint4(0, 0, 0, 0);
        if (col < m) y = *(const uint4 *)(acts.qs + col * K + (int64_t)b * 256 + g * 64 + r * 16);
        const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
        uint8_t *img = img0 + g * (int64_t)IW_BIMG;
        i_stg128(img + b_off, i_signed(u0, 0), i_signed(u0, 8), i_signed(u1, 0), i_signed(u1, 8));
        i_stg128(img + b_off + 128, i_signed(u2, 0), i_signed(u2, 8), i_signed(u3, 0), i_signed(u3, 8));
    }
    {
        // sums: thread (row tid / 4, pair tid % 4); the pair's four sums sit in slots 4 g .. 4 g + 3 of the 16
        const int scol_i = tid >> 2, g = tid & 3;
        const int64_t scol = cb * IW_COLS + scol_i;
        short4 bs = make_short4(0, 0, 0, 0);
        if (scol < m) bs = *(const short4 *)(acts.bsums + scol * (K / 16) + (int64_t)b * 16 + 4 * g);
        const uint32_t xy = i_h2_bits(__halves2half2(__short2half_rn(bs.x), __short2half_rn(bs.y)));
        const uint32_t zw = i_h2_bits(__halves2half2(__short2half_rn(bs.z), __short2half_rn(bs.w)));
        const bool odd = g & 1, second = g >> 1;
        const uint32_t v0 = odd ? 0u : xy, v1 = odd ? 0u : zw, v2 = odd ? xy : 0u, v3 = odd ? zw : 0u;
        uint8_t *bm = img0 + g * (int64_t)IW_BIMG + IW_B_BYTES + (scol_i >> 3) * 256 + (scol_i & 7) * 16;
        i_stg128(bm, second ? 0u : v0, second ? 0u : v1, second ? 0u : v2, second ? 0u : v3);
        i_stg128(bm + 128, second ? v0 : 0u, second ? v1 : 0u, second ? v2 : 0u, second ? v3 : 0u);
    }
    if (tid < IW_COLS) {
        const int64_t dcol = cb * IW_COLS + tid;
        daimg[(cb * nb + b) * IW_COLS + tid] = dcol < m ? acts.d[dcol * nb + b] : 0.0f;
    }
}

// 128 x 128 outputs per CTA.  Roles as in the 64-column kernel; epilogue warp w owns rows 32 (w % 4) .. + 31 and
// columns 32 (w / 4) .. + 31.
__global__ void __launch_bounds__(IM_THREADS, 1)
gemm_q4_K_tcgen05_img128_kernel(const uint8_t *__restrict__ tiles, const uint8_t *__restrict__ aimg, const uint8_t *__restrict__ bimg,
                                const float *__restrict__ daimg, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err) {
    extern __shared__ uint8_t iw_raw[];
    __shared__ IwBars bars;
    pdl_trigger();
    const uint32_t smem = (i_smem_u32(iw_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t rb = blockIdx.y, cb = blockIdx.x;
    const int64_t tile0 = rb * (IM_ROWS / TILE_ROWS), tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = cb * IW_COLS;
    const int np = 4 * nb;   // pipeline steps: sub-block pairs
    volatile int *abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < IW_STAGES; i++) {
            i_mbar_init(i_smem_u32(&bars.full[i]), 1);
            i_mbar_init(i_smem_u32(&bars.empty[i]), 1);
        }
        for (int i = 0; i < IM_TSTAGES; i++) {
            i_mbar_init(i_smem_u32(&bars.tfull[i]), 1);
            i_mbar_init(i_smem_u32(&bars.tempty[i]), IM_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == IM_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(i_smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;

    if (warp < IM_EPI_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(IM_REGS_EPI));
        pdl_wait();
        const int q = warp & 3, h4 = warp >> 2;
        const bool row_ok = tile0 + q < tiles_n;
        const bool any_col = col0 + 32 * h4 < m;
        const uint8_t *hdr = tiles + (row_ok ? tile0 + q : 0) * (int64_t)nb * 4608 + lane * 16;
        uint32_t dd_next = row_ok ? *(const uint32_t *)(hdr) : 0u;
        float dw = 0.0f, dmw = 0.0f;
        float sumf[32], summin[32];
#pragma unroll
        for (int c = 0; c < 32; c++) sumf[c] = summin[c] = 0.0f;
        const uint32_t trow0 = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(32 * h4);

        for (int e = 0; e < np; e++) {
            const int t = e % IM_TSTAGES, be = e >> 2;
            if ((e & 3) == 0) {
                dw = f16_bits_to_f32((uint16_t)(dd_next & 0xffffu));
                dmw = f16_bits_to_f32((uint16_t)(dd_next >> 16));
                if (be + 1 < nb && row_ok) dd_next = *(const uint32_t *)(hdr + (int64_t)(be + 1) * 4608);
            }
            if (!__all_sync(0xffffffffu, i_mbar_wait(i_smem_u32(&bars.tfull[t]), (uint32_t)(e / IM_TSTAGES) & 1u, abort_flag))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float4 *das = reinterpret_cast<const float4 *>(bars.da[be % IM_DA_SLOTS] + 32 * h4);
            const uint32_t trow = trow0 + (uint32_t)(t * 256);
            // four rounds of eight columns, the next round's loads in flight while this one's multiply-adds run:
            //   sumf = fma(f32(ig), d d_x, sumf);  summin = fma(f32(mg), dmin d_x, summin)
            float ig[2][8], mg[2][8];
            i_tmem_ld8f(ig[0], trow);
            i_tmem_ld8f(mg[0], trow + 128);
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const int c0 = 8 * r;
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r < 3) {
                    i_tmem_ld8f(ig[(r + 1) & 1], trow + (uint32_t)(c0 + 8));
                    i_tmem_ld8f(mg[(r + 1) & 1], trow + (uint32_t)(128 + c0 + 8));
                } else {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) i_mbar_arrive(i_smem_u32(&bars.tempty[t]));
                }
                if (any_col) {
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float4 dq = das[c0 / 4 + h];
                        const float dxs[4] = {dq.x, dq.y, dq.z, dq.w};
#pragma unroll
                        for (int c4 = 0; c4 < 4; c4++) {
                            const int c = 4 * h + c4;
                            sumf[c0 + c] = __fmaf_rn(ig[r & 1][c], __fmul_rn(dw, dxs[c4]), sumf[c0 + c]);
                            summin[c0 + c] = __fmaf_rn(mg[r & 1][c], __fmul_rn(dmw, dxs[c4]), summin[c0 + c]);
                        }
                    }
                }
            }
        }
        const int64_t row = (tile0 + q) * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 32; c++) {
                const int64_t col = col0 + 32 * h4 + c;
                if (col < m) dst[col * lddst + row] = __fsub_rn(sumf[c], summin[c]);
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(IM_REGS_CTL));
        pdl_wait();
        if (warp == IM_MMA_WARP) {
            if (lane == 0) {
                // per step: four K = 16 MMAs for ig, one for mg, N = 128
                for (int p = 0; p < np; p++) {
                    const int s = p % IW_STAGES, t = p % IM_TSTAGES;
                    if (!i_mbar_wait(i_smem_u32(&bars.full[s]), (uint32_t)(p / IW_STAGES) & 1u, abort_flag)) break;
                    if (!i_mbar_wait(i_smem_u32(&bars.tempty[t]), ((uint32_t)(p / IM_TSTAGES) & 1u) ^ 1u, abort_flag)) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_base = smem + (uint32_t)(s * IW_STAGE_BYTES), am_base = a_base + IW_A_BYTES;
                    const uint32_t b_base = a_base + IW_AIMG, bm_base = b_base + IW_B_BYTES;
                    i_issue_step128(tmem + (uint32_t)(t * 256), i_desc(a_base, 128, 1024), i_desc(b_base, 128, 1024), i_desc(am_base, 128, 256),
                                    i_desc(bm_base, 128, 256), IW_IDESC);
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(i_smem_u32(&bars.empty[s])) : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(i_smem_u32(&bars.tfull[t])) : "memory");
                }
            }
        } else if (warp == IM_LOAD_WARP && lane == 0) {
            const uint8_t *asrc = aimg + rb * np * (int64_t)IW_AIMG, *bsrc = bimg + cb * np * (int64_t)IW_BIMG;
            const float *dsrc = daimg + cb * nb * (int64_t)IW_COLS;
            int issued = -1;
            for (int p = 0; p < np; p++) {
                const int s = p % IW_STAGES;
                if (!i_mbar_wait(i_smem_u32(&bars.empty[s]), ((uint32_t)(p / IW_STAGES) & 1u) ^ 1u, abort_flag)) break;
                const uint32_t bar = i_smem_u32(&bars.full[s]), stage = smem + (uint32_t)(s * IW_STAGE_BYTES);
                const bool first = (p & 3) == 0;
                i_mbar_expect(bar, (uint32_t)(IW_STAGE_BYTES + (first ? IW_DA_BYTES : 0)));
                i_bulk_load(stage, asrc + (int64_t)p * IW_AIMG, IW_AIMG, bar);
                i_bulk_load(stage + IW_AIMG, bsrc + (int64_t)p * IW_BIMG, IW_BIMG, bar);
                // slot b % 4 is rewritten 16 steps later; the stage this step reuses (5 steps old) was released by
                // MMAs that had waited for the drain of every step of that older super-block
                if (first) i_bulk_load(i_smem_u32(bars.da[(p >> 2) % IM_DA_SLOTS]), dsrc + (int64_t)(p >> 2) * IW_COLS, IW_DA_BYTES, bar);
                issued = p;
            }
            if (*abort_flag && issued >= 0) i_mbar_wait(i_smem_u32(&bars.full[issued % IW_STAGES]), (uint32_t)(issued / IW_STAGES) & 1u, abort_flag);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == IM_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, IM_ERR_WAIT);
}

static int launch_images(bool wide, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_img_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IM_SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_img128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IW_SMEM_BYTES));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const int nb = (int)(k / GROUP_K);
    const int cols = wide ? IW_COLS : IM_COLS;
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t gx = (m + cols - 1) / cols, gy = (n + IM_ROWS - 1) / IM_ROWS;
    B200_REQUIRE(gx <= 65535 && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    // one block for the images of this mat-mul: weights, activations, activation scales
    // (per super-block and row or column block: 2 steps of 36 / 20 KB, or 4 steps of 20 / 20 KB)
    const size_t a_bytes = (size_t)gy * nb * (wide ? 4 * IW_AIMG : 2 * IM_AIMG), b_bytes = (size_t)gx * nb * (wide ? 4 * IW_BIMG : 2 * IM_BIMG);
    const size_t d_bytes = (size_t)gx * nb * (wide ? IW_DA_BYTES : IM_DA_BYTES);
    void *block = nullptr;
    rc = scratch_get_images(a_bytes + b_bytes + d_bytes, &block);
    if (rc != B200_STATUS_SUCCESS) return rc;
    uint8_t *aimg = (uint8_t *)block, *bimg = aimg + a_bytes;
    float *daimg = (float *)(bimg + b_bytes);
    const dim3 ga((unsigned)nb, (unsigned)gy), gb((unsigned)nb, (unsigned)gx), gg((unsigned)gx, (unsigned)gy);
    if (wide) {
        rc = launch_pdl(expand_q4_K_weights_pair_kernel, ga, dim3(IM_EXPAND_THREADS), (size_t)0, s, tiles, aimg, tiles_n, nb);
        if (rc != B200_STATUS_SUCCESS) return rc;
        rc = launch_pdl(expand_q8_K_acts_pair_kernel, gb, dim3(IM_EXPAND_THREADS), (size_t)0, s, acts, bimg, daimg, m, nb);
        if (rc != B200_STATUS_SUCCESS) return rc;
        return launch_pdl(gemm_q4_K_tcgen05_img128_kernel, gg, dim3(IM_THREADS), (size_t)IW_SMEM_BYTES, s, tiles, (const uint8_t *)aimg,
                          (const uint8_t *)bimg, (const float *)daimg, dst, lddst, n, nb, m, err);
    }
    rc = launch_pdl(expand_q4_K_weights_kernel, ga, dim3(IM_EXPAND_THREADS), (size_t)0, s, tiles, aimg, tiles_n, nb);
    if (rc != B200_STATUS_SUCCESS) return rc;
    rc = launch_pdl(expand_q8_K_acts_kernel, gb, dim3(IM_EXPAND_THREADS), (size_t)0, s, acts, bimg, daimg, m, nb);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_pdl(gemm_q4_K_tcgen05_img_kernel, gg, dim3(IM_THREADS), (size_t)IM_SMEM_BYTES, s, tiles, (const uint8_t *)aimg, (const uint8_t *)bimg,
                      (const float *)daimg, dst, lddst, n, nb, m, err);
}

int launch_gemm_tcgen05_img(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    return launch_images(false, n, k, m, tiles, acts, dst, lddst, s);
}
int launch_gemm_tcgen05_img128(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    return launch_images(true, n, k, m, tiles, acts, dst, lddst, s);
}

}  // namespace b200
