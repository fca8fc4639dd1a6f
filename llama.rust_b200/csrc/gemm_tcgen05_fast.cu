// Q4_K prompt mat-mul in the fast numerics mode (within 1e-5 of sum |w x| per output, not the CPU's bits): tcgen05 f16 MMAs
// that accumulate a whole 256-element super-block in tensor memory, one drain per super-block.
//
// The bit-exact two-pass kernels (gemm_tcgen05_img.cu) drain the accumulator once per sub-block pair, because the CPU's
// chain rounds there, and read their operands as unswizzled core matrices; both bound them far below the tensor cores'
// rate.  Here, per super-block b of an output (row n, activation row m),
//     ig = sum_j s_j sum_i w_ji x_ji      (s_j w <= 945, x: exact f16 operands; 256 products summed in f32 by the MMA)
//     mg = sum_j m_j (bsum_2j + bsum_2j+1) (mins and 16-element activation sums <= 2032: exact; sum < 2^24)
//     out += (d d_x) ig - (dmin d_x) mg
// which is the function the CPU computes (crates/ggml/src/repack.rs:1692-1768, tiled.rs) with the f32 additions in
// another order: ig itself may round once it passes 2^24, and the per-pair fused multiply-adds become one per super-block.
//
// Two passes, like the exact kernels: two small kernels expand the operands to f16 in exactly the shared-memory images the
// tensor core reads, the mat-mul kernel moves those images with bulk copies.  Images, per 128-row (or 128-column) block
// and super-block:
//   A  four pair columns [128 rows][64 f16], rows 128 bytes apart, 16-byte chunks XOR-swizzled with row % 8 (the 128-byte
//      swizzle of the matrix descriptor); within pair g the chunks are 4 p + 2 hi + half: 16-byte piece p of the pair's 32
//      nibble bytes, low | high nibbles, bytes (0,2,1,3,4,6,5,7 | 8 ..)                                    65536 B
//   Am [128 rows][16 f16], unswizzled core matrices: slots 2 j, 2 j + 1 = the min of sub-block j                 4096 B
//   B  the activation bytes in the same layout and K order                                                     65536 B
//   Bm [128 rows][16 f16]: the sixteen 16-element sums                                                          4096 B
//   da 128 f32 activation scales                                                                                 512 B
// Mat-mul kernel: 128 x 128 outputs per CTA; a pipeline step is half a super-block (two pair columns of A and of B,
// 64 KB, three stages); warp 9 (one thread) copies, warp 8 (one thread) issues 8 (+ 1 for the mins) MMAs per step into one
// of two tensor-memory stages (ig 128 columns, mg 128 columns), warps 0..7 drain: warp w owns rows 32 (w % 4) .. + 31 (its
// tensor-memory lanes) and columns 64 (w / 4) .. + 63.  Every wait is bounded; a wait that runs out raises the CTA's abort
// flag and the device error word.
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int FQ_ROWS = 128, FQ_COLS = 128;
constexpr int FQ_EPI_WARPS = 8, FQ_MMA_WARP = 8, FQ_LOAD_WARP = 9;
constexpr int FQ_PROD_WARP0 = 12, FQ_PROD_WARPS = 8;   // FUSED: the warps that unpack the CTA's weights (a row's half step per thread)
constexpr int FQ_THREADS = 20 * 32;          // five warp groups: two of epilogue warps, the two single-thread roles, two of producers
constexpr int FQ_REGS_EPI = 144, FQ_REGS_CTL = 40, FQ_REGS_PROD = 64;   // 2 x 144 + 40 + 2 x 64 = 456 <= 5 x 96
constexpr int FQ_EXPAND_THREADS = 512;
constexpr int FQ_PAIR_BYTES = FQ_ROWS * 128; // one pair column: 16384
constexpr int FQ_A_BYTES = 4 * FQ_PAIR_BYTES, FQ_M_BYTES = FQ_ROWS * 32, FQ_DA_BYTES = FQ_COLS * 4;
constexpr int FQ_AIMG = FQ_A_BYTES + FQ_M_BYTES;                 // 69632
constexpr int FQ_BIMG = FQ_A_BYTES + FQ_M_BYTES + FQ_DA_BYTES;   // 70144
constexpr int FQ_STAGES = 3, FQ_TSTAGES = 2, FQ_MSLOTS = 2, FQ_DA_SLOTS = 4;
constexpr int FQ_HALF = 2 * FQ_PAIR_BYTES;                       // 32768: half a super-block of one operand
constexpr int FQ_STAGE_BYTES = 2 * FQ_HALF;                      // 65536
constexpr int FQ_SMEM_BYTES = FQ_STAGES * FQ_STAGE_BYTES + FQ_MSLOTS * 2 * FQ_M_BYTES + 1024;   // 214016
constexpr uint32_t FQ_WAIT_LIMIT = 1u << 22;
constexpr int FQ_ERR_WAIT = 4;
// kind::f16 instruction descriptor: f32 accumulator, f16 x f16, both operands K-major, N = 128, M = 128
constexpr uint32_t FQ_IDESC = (1u << 4) | ((uint32_t)(FQ_COLS >> 3) << 17) | ((uint32_t)(FQ_ROWS >> 4) << 24);

__device__ __forceinline__ uint32_t q_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// shared-memory matrix descriptors (version 1 in bit 46).  Unswizzled: K-adjacent core matrices lbo bytes apart, 8-row
// groups sbo bytes apart.  128-byte swizzle (layout type 2 in bits 61..63): rows 128 bytes apart, 8-row groups 1024 bytes
// apart, the leading offset unused; a K = 16 step moves the start address by 32 bytes inside the swizzle atom.
__device__ __forceinline__ uint64_t q_desc_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint64_t q_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void q_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void q_mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void q_mbar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy, one destination CTA; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void q_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool q_mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < FQ_WAIT_LIMIT; it++) {
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
// 32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void q_tmem_ld32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void q_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, int accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc), "l"(bdesc),
                 "r"(FQ_IDESC), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ uint32_t q_h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 q_bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
// low nibbles of bytes 0 and 2 of the word, times the scale: (1024 + w) s - 1024 s, one rounding, exact
__device__ __forceinline__ uint32_t q_scaled_lo(uint32_t word, __half2 s2, __half2 c2) {
    return q_h2_bits(__hfma2(q_bits_h2((word & 0x000f000fu) | 0x64006400u), s2, c2));
}
// high nibbles, left where they are: (1024 + 16 w) (s / 16) - 64 s; s / 16 and 64 s are exact in f16
__device__ __forceinline__ uint32_t q_scaled_hi(uint32_t word, __half2 s16, __half2 c16) {
    return q_h2_bits(__hfma2(q_bits_h2((word & 0x00f000f0u) | 0x64006400u), s16, c16));
}
// an integer 0 .. 1023 in both halves: (1024 + v) - 1024
__device__ __forceinline__ __half2 q_small2(uint32_t v) { return __hsub2(q_bits_h2(0x64006400u | v | (v << 16)), q_bits_h2(0x64006400u)); }
// signed bytes 0 and 2 of the word (after the sign flip u = y ^ 0x80): (1024 + u) - 1152, exact
__device__ __forceinline__ uint32_t q_signed(uint32_t u, int shift) {
    return q_h2_bits(__hsub2(q_bits_h2(((u >> shift) & 0x00ff00ffu) | 0x64006400u), __float2half2_rn(1152.0f)));
}
__device__ __forceinline__ void q_stg128(uint8_t *p, uint32_t x, uint32_t y, uint32_t z, uint32_t w) { *reinterpret_cast<uint4 *>(p) = make_uint4(x, y, z, w); }

// profiling aid (B200_GEMM_FAST_PROFILE=1): SM clocks one thread of each role of CTA (0, 0) spends waiting at each of its
// barriers and working, summed over the steps: [0] epilogue warp 0 waiting for the accumulator, [1] draining it; [2] MMA
// thread waiting for a stage, [3] for a tensor-memory stage, [4] issuing; [5] loader waiting for a free stage, [6] issuing;
// [7] producer warp 12 waiting for a free stage, [8] converting; [9] the CTA's whole run
__device__ unsigned long long g_fq_prof[16];
#define FQ_MARK(k)                                            \
    do {                                                      \
        if (prof) {                                           \
            const long long t_now = clock64();                \
            pacc[k] += (unsigned long long)(t_now - t_prev);  \
            t_prev = t_now;                                   \
        }                                                     \
    } while (0)

struct alignas(16) FqBars {
    uint64_t full[FQ_STAGES], empty[FQ_STAGES], tfull[FQ_TSTAGES], tempty[FQ_TSTAGES];
    float da[FQ_DA_SLOTS][FQ_COLS];
    uint32_t tmem_base;
    int abort_flag;
};

}  // namespace

// Weights of one 128-row block and one super-block -> its A and Am images.  Warp (tt, aj): row (tile tt, lane), 16-byte
// pieces aj and 4 + aj of the row's 128 nibble bytes.
__global__ void __launch_bounds__(FQ_EXPAND_THREADS) expand_q4_K_weights_fast_kernel(const uint8_t *__restrict__ tiles, uint8_t *aimg, int64_t tiles_n, int nb) {
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
    uint8_t *img = aimg + (rb * nb + b) * (int64_t)FQ_AIMG;
    if (aj == 0) {
        const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
        uint32_t mins[8];
#pragma unroll
        for (int j = 0; j < 8; j++) mins[j] = q_h2_bits(q_small2(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu));
        uint8_t *am = img + FQ_A_BYTES + (prow >> 3) * 256 + (prow & 7) * 16;
        q_stg128(am, mins[0], mins[1], mins[2], mins[3]);
        q_stg128(am + 128, mins[4], mins[5], mins[6], mins[7]);
    }
    // piece within the pair pp = aj % 2: chunks 4 pp + {0, 1 low | 2, 3 high}, each at (chunk ^ row % 8)
    const int sw = prow & 7;
    uint8_t *rowp = img + prow * 128;
#pragma unroll
    for (int hs = 0; hs < 2; hs++) {
        // piece c = 4 hs + aj of the row: pair g = c / 2 (sub-blocks 2 g, 2 g + 1)
        const int g = 2 * hs + (aj >> 1);
        const uint4 w = wq[hs];
        const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
        const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
        const __half2 sl = q_small2(s_lo), sh = q_small2(s_hi);
        // -1024 s <= 64512 in magnitude: a multiple of 1024 below 65504, exact in f16
        const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
        const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
        const uint32_t x8 = w.x >> 8, y8 = w.y >> 8, z8 = w.z >> 8, w8 = w.w >> 8;   // bytes 1 and 3
        uint8_t *dstp = rowp + g * FQ_PAIR_BYTES;
        const int c0 = 4 * (aj & 1);
        q_stg128(dstp + (((c0 + 0) ^ sw) << 4), q_scaled_lo(w.x, sl, cl), q_scaled_lo(x8, sl, cl), q_scaled_lo(w.y, sl, cl), q_scaled_lo(y8, sl, cl));
        q_stg128(dstp + (((c0 + 1) ^ sw) << 4), q_scaled_lo(w.z, sl, cl), q_scaled_lo(z8, sl, cl), q_scaled_lo(w.w, sl, cl), q_scaled_lo(w8, sl, cl));
        q_stg128(dstp + (((c0 + 2) ^ sw) << 4), q_scaled_hi(w.x, sh16, ch), q_scaled_hi(x8, sh16, ch), q_scaled_hi(w.y, sh16, ch), q_scaled_hi(y8, sh16, ch));
        q_stg128(dstp + (((c0 + 3) ^ sw) << 4), q_scaled_hi(w.z, sh16, ch), q_scaled_hi(z8, sh16, ch), q_scaled_hi(w.w, sh16, ch), q_scaled_hi(w8, sh16, ch));
    }
}

// Q8_K activations of one 128-row block and one super-block -> its B and Bm images and the scales.
__global__ void __launch_bounds__(FQ_EXPAND_THREADS) expand_q8_K_acts_fast_kernel(ActView acts, uint8_t *bimg, int64_t m, int nb) {
    pdl_trigger();
    pdl_wait();   // the activations come from the previous kernel
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int b = blockIdx.x;
    const int64_t cb = blockIdx.y, K = acts.k;
    uint8_t *img = bimg + (cb * nb + b) * (int64_t)FQ_BIMG;
    // a warp reads 64 contiguous bytes (one pair) of 8 activation rows
    const int bc = warp * 8 + (lane & 7), r = lane >> 3;
    const int64_t col = cb * FQ_COLS + bc;
    // piece r of the pair: (low p0, low p1, high p0, high p1) -> chunks 4 p + 2 hi + {0, 1}
    const int c0 = 4 * (r & 1) + 2 * (r >> 1), sw = bc & 7;
    uint8_t *rowp = img + bc * 128;
#pragma unroll
    for (int g = 0; g < 4; g++) {
        uint4 y = make_uint4(0, 0, 0, 0);
        if (col < m) y = *(const uint4 *)(acts.qs + col * K + (int64_t)b * 256 + g * 64 + r * 16);
        // a row past the end holds zeros: 0x80 after the flip, 128 - 128 = 0
        const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
        uint8_t *dstp = rowp + g * FQ_PAIR_BYTES;
        q_stg128(dstp + (((c0 + 0) ^ sw) << 4), q_signed(u0, 0), q_signed(u0, 8), q_signed(u1, 0), q_signed(u1, 8));
        q_stg128(dstp + (((c0 + 1) ^ sw) << 4), q_signed(u2, 0), q_signed(u2, 8), q_signed(u3, 0), q_signed(u3, 8));
    }
    if (tid < 2 * FQ_COLS) {
        // sums: thread (row tid / 2, half tid % 2): eight 16-element sums -> one core-matrix row
        const int scol_i = tid >> 1, kc = tid & 1;
        const int64_t scol = cb * FQ_COLS + scol_i;
        short4 b0 = make_short4(0, 0, 0, 0), b1 = b0;
        if (scol < m) {
            const short4 *bp = (const short4 *)(acts.bsums + scol * (K / 16) + (int64_t)b * 16 + 8 * kc);
            b0 = bp[0];
            b1 = bp[1];
        }
        uint8_t *bm = img + FQ_A_BYTES + (scol_i >> 3) * 256 + (scol_i & 7) * 16 + kc * 128;
        q_stg128(bm, q_h2_bits(__halves2half2(__short2half_rn(b0.x), __short2half_rn(b0.y))), q_h2_bits(__halves2half2(__short2half_rn(b0.z), __short2half_rn(b0.w))),
                 q_h2_bits(__halves2half2(__short2half_rn(b1.x), __short2half_rn(b1.y))), q_h2_bits(__halves2half2(__short2half_rn(b1.z), __short2half_rn(b1.w))));
    } else if (tid < 3 * FQ_COLS) {
        const int dcol_i = tid - 2 * FQ_COLS;
        const int64_t dcol = cb * FQ_COLS + dcol_i;
        reinterpret_cast<float *>(img + FQ_A_BYTES + FQ_M_BYTES)[dcol_i] = dcol < m ? acts.d[dcol * nb + b] : 0.0f;
    }
}

// FUSED: no weight images; warps 12..19 unpack the 128 rows' nibbles of every step straight into the stage (and the mins
// into their slot), so the weights cross the L2 as 0.5625 bytes each instead of 2
template <bool FUSED>
__global__ void __launch_bounds__(FQ_THREADS, 1)
gemm_q4_K_tcgen05_fast_kernel(const uint8_t *__restrict__ tiles, const uint8_t *__restrict__ aimg, const uint8_t *__restrict__ bimg, float *dst,
                              int64_t lddst, int64_t n, int nb, int64_t m, int *err, int profile) {
    extern __shared__ uint8_t fq_raw[];
    __shared__ FqBars bars;
    pdl_trigger();
    const uint32_t smem = (q_smem_u32(fq_raw) + 1023u) & ~1023u;
    const uint32_t mslots = smem + (uint32_t)(FQ_STAGES * FQ_STAGE_BYTES);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t rb = blockIdx.y, cb = blockIdx.x;
    const int64_t tile0 = rb * (FQ_ROWS / TILE_ROWS), tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = cb * FQ_COLS;
    const int np = 2 * nb;   // pipeline steps: half super-blocks
    volatile int *abort_flag = &bars.abort_flag;
    const bool prof = profile && blockIdx.x == 0 && blockIdx.y == 0 && lane == 0;
    long long t_prev = clock64();
    const long long t_start = t_prev;
    unsigned long long pacc[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // kept in registers, written once at the end

    if (threadIdx.x == 0) {
        for (int i = 0; i < FQ_STAGES; i++) {
            q_mbar_init(q_smem_u32(&bars.full[i]), FUSED ? 1 + FQ_PROD_WARPS : 1);   // the loader's arrive + the bytes it announced (+ the producer warps)
            q_mbar_init(q_smem_u32(&bars.empty[i]), 1);   // the MMA thread's commit
        }
        for (int i = 0; i < FQ_TSTAGES; i++) {
            q_mbar_init(q_smem_u32(&bars.tfull[i]), 1);
            q_mbar_init(q_smem_u32(&bars.tempty[i]), FQ_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == FQ_MMA_WARP) {
        // all 512 columns: the CTA's shared memory already keeps a second CTA off this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(q_smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;

    if (warp < FQ_EPI_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FQ_REGS_EPI));
        pdl_wait();   // the images are the previous kernels' output, and the previous mat-mul may still be reading dst's producers
        const int q = warp & 3, h = warp >> 2;
        const bool row_ok = tile0 + q < tiles_n;
        const bool any_col = col0 + 64 * h < m;
        // (d, dmin) of this thread's row, one word per super-block, fetched one super-block ahead
        const uint8_t *hdr = tiles + (row_ok ? tile0 + q : 0) * (int64_t)nb * 4608 + lane * 16;
        uint32_t dd_next = row_ok ? *(const uint32_t *)(hdr) : 0u;
        float acc[64];
#pragma unroll
        for (int c = 0; c < 64; c++) acc[c] = 0.0f;
        const uint32_t trow0 = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(64 * h);
        for (int b = 0; b < nb; b++) {
            const int t = b % FQ_TSTAGES;
            const float dw = f16_bits_to_f32((uint16_t)(dd_next & 0xffffu)), dmw = -f16_bits_to_f32((uint16_t)(dd_next >> 16));
            if (b + 1 < nb && row_ok) dd_next = *(const uint32_t *)(hdr + (int64_t)(b + 1) * 4608);
            if (warp == 0) FQ_MARK(1);
            if (!__all_sync(0xffffffffu, q_mbar_wait(q_smem_u32(&bars.tfull[t]), (uint32_t)(b / FQ_TSTAGES) & 1u, abort_flag))) break;
            if (warp == 0) FQ_MARK(0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float4 *das = reinterpret_cast<const float4 *>(bars.da[b % FQ_DA_SLOTS] + 64 * h);
            const uint32_t trow = trow0 + (uint32_t)(t * 256);
            // two rounds of 32 columns: one tensor-memory round trip each for ig and mg, then per column
            //   acc += d_x (d ig - dmin mg)
            uint32_t ig[32], mg[32];
#pragma unroll
            for (int r = 0; r < 2; r++) {
                q_tmem_ld32(ig, trow + (uint32_t)(32 * r));
                q_tmem_ld32(mg, trow + (uint32_t)(128 + 32 * r));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (r == 1) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.tempty[t]));
                }
                if (any_col) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; c4++) {
                        const float4 dq = das[8 * r + c4];
                        const float dxs[4] = {dq.x, dq.y, dq.z, dq.w};
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            const float tsum = fmaf(__uint_as_float(mg[4 * c4 + c]), dmw, __uint_as_float(ig[4 * c4 + c]) * dw);
                            acc[32 * r + 4 * c4 + c] = fmaf(tsum, dxs[c], acc[32 * r + 4 * c4 + c]);
                        }
                    }
                }
            }
        }
        const int64_t row = (tile0 + q) * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 64; c++) {
                const int64_t col = col0 + 64 * h + c;
                if (col < m) dst[col * lddst + row] = acc[c];
            }
        }
    } else if (warp >= FQ_PROD_WARP0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FQ_REGS_PROD));
        if constexpr (FUSED) {
            // thread = (row (tile tt, lane), pair column hh of the step): per step the two 16-byte pieces 4 hs + 2 hh, + 1 of the
            // row's 128 nibble bytes, loaded one step ahead (the weights do not depend on the previous kernel)
            const int pw = warp - FQ_PROD_WARP0, tt = pw & 3, hh = pw >> 2, prow = tt * 32 + lane, sw = prow & 7;
            const bool tile_ok = tile0 + tt < tiles_n;
            const uint8_t *src = tiles + (tile_ok ? tile0 + tt : 0) * (int64_t)nb * 4608 + lane * 16;
            uint8_t *stage0 = fq_raw + (smem - q_smem_u32(fq_raw)) + hh * FQ_PAIR_BYTES + prow * 128;
            uint8_t *am0 = fq_raw + (mslots - q_smem_u32(fq_raw)) + (prow >> 3) * 256 + (prow & 7) * 16;
            uint4 hd = make_uint4(0, 0, 0, 0), hd_next = hd, w[2], wn[2];
            wn[0] = wn[1] = hd;
            if (tile_ok) {
                hd_next = *(const uint4 *)src;
#pragma unroll
                for (int i = 0; i < 2; i++) wn[i] = ld_stream16(src + 512 + (2 * hh + i) * 512);
            }
            for (int p = 0; p < np; p++) {
                const int s = p % FQ_STAGES, b = p >> 1, hs = p & 1;
                w[0] = wn[0];
                w[1] = wn[1];
                if (hs == 0) hd = hd_next;
                if (p + 1 < np && tile_ok) {
                    const uint8_t *nx = src + (int64_t)((p + 1) >> 1) * 4608;
                    if (hs == 1) hd_next = *(const uint4 *)nx;
#pragma unroll
                    for (int i = 0; i < 2; i++) wn[i] = ld_stream16(nx + 512 + (4 * (hs ^ 1) + 2 * hh + i) * 512);
                }
                if (warp == FQ_PROD_WARP0) FQ_MARK(8);
                if (!__all_sync(0xffffffffu, q_mbar_wait(q_smem_u32(&bars.empty[s]), ((uint32_t)(p / FQ_STAGES) & 1u) ^ 1u, abort_flag))) break;
                if (warp == FQ_PROD_WARP0) FQ_MARK(7);
                if (profile == 2) {
                    __syncwarp();
                    if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.full[s]));
                    continue;
                }
                if (hs == 0 && hh == 0) {
                    // the mins slot of super-block b - 2 is free: see the loader
                    const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
                    uint32_t mins[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) mins[j] = q_h2_bits(q_small2(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu));
                    uint8_t *am = am0 + (b % FQ_MSLOTS) * 2 * FQ_M_BYTES;
                    q_stg128(am, mins[0], mins[1], mins[2], mins[3]);
                    q_stg128(am + 128, mins[4], mins[5], mins[6], mins[7]);
                }
                {
                    // pair g = 2 hs + hh (sub-blocks 2 g, 2 g + 1): the step's pair column hh
                    const int g = 2 * hs + hh;
                    const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
                    const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
                    const __half2 sl = q_small2(s_lo), sh = q_small2(s_hi);
                    const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
                    const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
                    uint8_t *dstp = stage0 + s * FQ_STAGE_BYTES;
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const uint4 v = w[i];
                        const uint32_t x8 = v.x >> 8, y8 = v.y >> 8, z8 = v.z >> 8, w8 = v.w >> 8;   // bytes 1 and 3
                        const int c0 = 4 * i;
                        q_stg128(dstp + (((c0 + 0) ^ sw) << 4), q_scaled_lo(v.x, sl, cl), q_scaled_lo(x8, sl, cl), q_scaled_lo(v.y, sl, cl), q_scaled_lo(y8, sl, cl));
                        q_stg128(dstp + (((c0 + 1) ^ sw) << 4), q_scaled_lo(v.z, sl, cl), q_scaled_lo(z8, sl, cl), q_scaled_lo(v.w, sl, cl), q_scaled_lo(w8, sl, cl));
                        q_stg128(dstp + (((c0 + 2) ^ sw) << 4), q_scaled_hi(v.x, sh16, ch), q_scaled_hi(x8, sh16, ch), q_scaled_hi(v.y, sh16, ch), q_scaled_hi(y8, sh16, ch));
                        q_stg128(dstp + (((c0 + 3) ^ sw) << 4), q_scaled_hi(v.z, sh16, ch), q_scaled_hi(z8, sh16, ch), q_scaled_hi(v.w, sh16, ch), q_scaled_hi(w8, sh16, ch));
                    }
                }
                // the stores (generic proxy) before the tensor core's reads (async proxy), then the warp's arrival
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.full[s]));
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FQ_REGS_CTL));
        pdl_wait();
    if (warp == FQ_MMA_WARP) {
        if (lane == 0) {
            for (int p = 0; p < np; p++) {
                const int s = p % FQ_STAGES, b = p >> 1, hs = p & 1, t = b % FQ_TSTAGES;
                FQ_MARK(4);
                if (!q_mbar_wait(q_smem_u32(&bars.full[s]), (uint32_t)(p / FQ_STAGES) & 1u, abort_flag)) break;
                FQ_MARK(2);
                if (hs == 0 && !q_mbar_wait(q_smem_u32(&bars.tempty[t]), ((uint32_t)(b / FQ_TSTAGES) & 1u) ^ 1u, abort_flag)) break;
                FQ_MARK(3);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_base = smem + (uint32_t)(s * FQ_STAGE_BYTES), b_base = a_base + FQ_HALF;
                const uint32_t d_ig = tmem + (uint32_t)(t * 256);
                if (hs == 0) {
                    const uint32_t am = mslots + (uint32_t)((b % FQ_MSLOTS) * 2 * FQ_M_BYTES);
                    q_mma(d_ig + 128, q_desc_plain(am, 128, 256), q_desc_plain(am + FQ_M_BYTES, 128, 256), 0);
                }
                const uint64_t ad = q_desc_sw128(a_base), bd = q_desc_sw128(b_base);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    // pair column i / 4 (16384 bytes on), K = 16 step i % 4 (32 bytes on); descriptor addresses count 16 bytes
                    const uint64_t off = (uint64_t)((i >> 2) * (FQ_PAIR_BYTES >> 4) + (i & 3) * 2);
                    q_mma(d_ig, ad + off, bd + off, (hs | i) != 0);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(q_smem_u32(&bars.empty[s])) : "memory");
                if (hs == 1)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(q_smem_u32(&bars.tfull[t])) : "memory");
            }
        }
    } else if (warp == FQ_LOAD_WARP && lane == 0) {
        const uint8_t *asrc = aimg + rb * nb * (int64_t)FQ_AIMG, *bsrc = bimg + cb * nb * (int64_t)FQ_BIMG;
        int issued = -1;
        for (int p = 0; p < np; p++) {
            const int s = p % FQ_STAGES, b = p >> 1, hs = p & 1;
            FQ_MARK(6);
            if (!q_mbar_wait(q_smem_u32(&bars.empty[s]), ((uint32_t)(p / FQ_STAGES) & 1u) ^ 1u, abort_flag)) break;
            FQ_MARK(5);
            const uint32_t bar = q_smem_u32(&bars.full[s]), stage = smem + (uint32_t)(s * FQ_STAGE_BYTES);
            const uint8_t *ab = FUSED ? nullptr : asrc + (int64_t)b * FQ_AIMG, *bb = bsrc + (int64_t)b * FQ_BIMG;
            if (profile == 2) {   // measurement only: no operand traffic at all (the outputs are garbage)
                q_mbar_arrive(bar);
                continue;
            }
            q_mbar_expect(bar, (uint32_t)((FUSED ? FQ_HALF : FQ_STAGE_BYTES) + (hs == 0 ? (FUSED ? 1 : 2) * FQ_M_BYTES + FQ_DA_BYTES : 0)));
            if (!FUSED) q_bulk_load(stage, ab + hs * FQ_HALF, FQ_HALF, bar);
            q_bulk_load(stage + FQ_HALF, bb + hs * FQ_HALF, FQ_HALF, bar);
            if (hs == 0) {
                // the mins slot of super-block b - 2 and the scale slot of b - 4 are free: the stage this step reuses was
                // released by MMAs issued after the drain of super-block b - 2 had ended
                const uint32_t ms = mslots + (uint32_t)((b % FQ_MSLOTS) * 2 * FQ_M_BYTES);
                if (!FUSED) q_bulk_load(ms, ab + FQ_A_BYTES, FQ_M_BYTES, bar);
                q_bulk_load(ms + FQ_M_BYTES, bb + FQ_A_BYTES, FQ_M_BYTES, bar);
                q_bulk_load(q_smem_u32(bars.da[b % FQ_DA_SLOTS]), bb + FQ_A_BYTES + FQ_M_BYTES, FQ_DA_BYTES, bar);
            }
            issued = p;
        }
        // a CTA that gives up still waits (bounded) for the copies it has in flight
        if (*abort_flag && issued >= 0) q_mbar_wait(q_smem_u32(&bars.full[issued % FQ_STAGES]), (uint32_t)(issued / FQ_STAGES) & 1u, abort_flag);
    }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FQ_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, FQ_ERR_WAIT);
    if (prof) {
#pragma unroll
        for (int i = 0; i < 9; i++)
            if (pacc[i]) atomicAdd(&g_fq_prof[i], pacc[i]);
        if (threadIdx.x == 0) atomicAdd(&g_fq_prof[9], (unsigned long long)(clock64() - t_start));
    }
}

// the clocks of the profiled launches so far (see g_fq_prof); reading clears them
int gemm_fast_profile(unsigned long long *out, int n) {
    if (n > 16) n = 16;
    B200_CUDA(cudaMemcpyFromSymbol(out, g_fq_prof, (size_t)n * sizeof(unsigned long long)));
    static const unsigned long long zeros[16] = {0};
    B200_CUDA(cudaMemcpyToSymbol(g_fq_prof, zeros, sizeof(zeros)));
    return B200_STATUS_SUCCESS;
}

int launch_gemm_q4_K_fast(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_fast_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FQ_SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_fast_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FQ_SMEM_BYTES));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    // B200_GEMM_FAST_FUSED=0: the weights through an image of their own (expanded by a kernel before the mat-mul) instead of
    // the mat-mul's producer warps (read per call)
    const char *ev = getenv("B200_GEMM_FAST_FUSED");
    const bool fused = !(ev && ev[0] == '0');
    const char *pv = getenv("B200_GEMM_FAST_PROFILE");
    const int profile = pv && pv[0] >= '1' && pv[0] <= '2' ? pv[0] - '0' : 0;   // 2: no operand traffic, garbage out (measurement of the MMA / drain rate alone)
    const int nb = (int)(k / GROUP_K);
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t gx = (m + FQ_COLS - 1) / FQ_COLS, gy = (n + FQ_ROWS - 1) / FQ_ROWS;
    B200_REQUIRE(gx <= 65535 && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    const size_t a_bytes = fused ? 0 : (size_t)gy * nb * FQ_AIMG, b_bytes = (size_t)gx * nb * FQ_BIMG;
    void *block = nullptr;
    rc = scratch_get_images(a_bytes + b_bytes, &block);
    if (rc != B200_STATUS_SUCCESS) return rc;
    uint8_t *aimg = (uint8_t *)block, *bimg = aimg + a_bytes;
    const dim3 ga((unsigned)nb, (unsigned)gy), gb((unsigned)nb, (unsigned)gx), gg((unsigned)gx, (unsigned)gy);
    if (!fused) {
        rc = launch_pdl(expand_q4_K_weights_fast_kernel, ga, dim3(FQ_EXPAND_THREADS), (size_t)0, s, tiles, aimg, tiles_n, nb);
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    rc = launch_pdl(expand_q8_K_acts_fast_kernel, gb, dim3(FQ_EXPAND_THREADS), (size_t)0, s, acts, bimg, m, nb);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (fused)
        return launch_pdl(gemm_q4_K_tcgen05_fast_kernel<true>, gg, dim3(FQ_THREADS), (size_t)FQ_SMEM_BYTES, s, tiles, (const uint8_t *)aimg,
                          (const uint8_t *)bimg, dst, lddst, n, nb, m, err, profile);
    return launch_pdl(gemm_q4_K_tcgen05_fast_kernel<false>, gg, dim3(FQ_THREADS), (size_t)FQ_SMEM_BYTES, s, tiles, (const uint8_t *)aimg, (const uint8_t *)bimg,
                      dst, lddst, n, nb, m, err, profile);
}

}  // namespace b200
