// Q4_K (and Q6_K, below) prompt mat-mul in the fast numerics mode (within 1e-5 of sum |w x| per output, not the CPU's bits):
// tcgen05 f16 MMAs that accumulate a whole 256-element super-block, mins included, in ONE tensor-memory accumulator, drained
// once per super-block.
//
// The bit-exact two-pass kernels (gemm_tcgen05_img.cu) drain two accumulators once per sub-block pair, because the CPU's chain
// rounds there, and read their operands as unswizzled core matrices; both bound them far below the tensor cores' rate.
// Measured here: an M = 128, K = 16 MMA takes 128 cycles whatever N <= 256 is, so only N = 256 runs the tensor core at its
// rate, and 512 tensor-memory columns hold two stages of N = 256 only if a super-block needs one accumulator.  So, per
// super-block b of an output (row n, activation row m), with d, dmin the row's block scales and rho = dmin / d,
//     acc = sum_j s_j sum_i w_ji x_ji  -  sum_j (rho m_j) (bsum_2j + bsum_2j+1)
//     out += d_x (d acc)
// s_j w (<= 945), x and the 16-element activation sums (<= 2032) are exact f16 operands; rho m_j is an f32 carried as two
// f16 operands (high part + remainder, 22 bits) against the sums repeated; the MMA adds the 256 + 32 products in f32.  This
// is the function the CPU computes (crates/ggml/src/repack.rs:1692-1768, tiled.rs) with the f32 operations in another order.
// A row whose d is zero, or whose rho m_j could leave the f16 range (rho > 952), gets zero mins operands for that
// super-block and the drain subtracts d_x dmin sum_j m_j bsum_j for it on the CUDA cores instead (read back from the
// activations' own sums; seen on no real tensor, kept exact all the same).
//
// Operands.  The activations are expanded once per mat-mul by a small kernel to the shared-memory images the tensor core
// reads, per block of NC (128 or 256) activation rows and super-block:
//   B   four pair columns [NC rows][64 f16], rows 128 bytes apart, 16-byte chunks XOR-swizzled with row % 8 (the 128-byte
//       swizzle of the matrix descriptor); within pair g the chunks are 4 p + 2 hi + half: 16-byte piece p of the pair's 32
//       nibble bytes, low | high nibbles, bytes (0,2,1,3,4,6,5,7 | 8 ..)
//   Bm  [NC rows][32 f16], unswizzled core matrices: the sixteen 16-element sums, twice
//   da  NC f32 activation scales
// and move with bulk copies.  The weights take no image: four producer warps (a row per thread) unpack the 128 rows' nibbles
// of every step straight into the stage in the same layout (A), and at the first step of a super-block the mins operand Am
// [128 rows][32 f16] (slots 2 j, 2 j + 1 = high part of -rho m_j, slots 16 + 2 j, + 1 = the remainder), so the weights cross
// the L2 as 0.5625 bytes each.
// Mat-mul kernel: tiles of 128 x NC outputs; a pipeline step is one pair column (K = 64: 16 KB of A, NC x 128 bytes of B);
// warp 9 (one thread) copies, warp 8 (one thread) issues 4 (+ 2 for the mins) MMAs per step into one of two tensor-memory
// stages of NC columns, warps 0..7 drain: warp w owns rows 32 (w % 4) .. + 31 (its tensor-memory lanes) and columns
// NC / 2 (w / 4) .. + NC / 2 - 1, warps 12..15 produce A.  A CTA walks a contiguous run of (tile, super-block) units (see
// FqSplit); up to three matrices over the same activations share a launch (FqMats).  Every wait is bounded; a wait that
// runs out raises the CTA's abort flag and the device error word.
#include <cuda_fp16.h>

#include <cmath>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int FQ_ROWS = 128;
constexpr int FQ_EPI_WARPS = 8, FQ_MMA_WARP = 8, FQ_LOAD_WARP = 9;
constexpr int FQ_PROD_WARP0 = 12, FQ_PROD_WARPS = 4;
constexpr int FQ_THREADS = 16 * 32;          // four warp groups: two of epilogue warps, the two single-thread roles, the producers
constexpr int FQ_REGS_EPI = 200, FQ_REGS_CTL = 40, FQ_REGS_PROD = 72;   // 2 x 200 + 40 + 72 = 512 = 4 x 128
constexpr int FQ_EXPAND_THREADS = 512;
constexpr int FQ_A_STEP = FQ_ROWS * 128;     // one pair column of the weights: 16384
constexpr int FQ_AM_BYTES = FQ_ROWS * 64;    // 8192
constexpr int FQ_TSTAGES = 2, FQ_DA_SLOTS = 4;
constexpr uint32_t FQ_WAIT_LIMIT = 1u << 22;
constexpr int FQ_ERR_WAIT = 4;
constexpr float FQ_RHO_MAX = 952.0f;         // 63 rho stays below 60000 < 65504

// Q6_K (the same kernel, Q6 = true): no mins; a weight is s (q - 32) with an int8 scale per 16 elements, up to 4096 in
// magnitude and so not always an f16 integer.  It goes in as two exact operands, s (8 (q >> 3) - 32) (a multiple of 8 up to
// 4096) and s (q & 7) (up to 896), multiplied against the same activation image: twice the MMAs, one accumulator.  A step is
// the 64 elements one (128-element half n, 16-byte piece l16) of the block's ql / qh bytes yields: the four 16-element runs
// 128 n + 32 r + 16 l16 .. + 15, r = 0 .. 3, each under its own scale; chunk c of a step's image row holds elements
// 8 (c % 2) .. + 7 of run c / 2 (bytes (0,2,1,3,4,6,5,7)).
template <int NC, bool Q6>
struct FqCfg {
    static constexpr int A_STEP = (Q6 ? 2 : 1) * FQ_A_STEP;       // Q6_K: the high-part tile, then the low-part tile
    static constexpr int B_STEP = NC * 128;                       // one step of the activations
    static constexpr int BM_BYTES = Q6 ? 0 : NC * 64, DA_BYTES = NC * 4;
    static constexpr int AM_BYTES = Q6 ? 0 : FQ_AM_BYTES;
    static constexpr int BIMG = 4 * B_STEP + BM_BYTES + DA_BYTES; // per (column block, super-block)
    static constexpr int STAGE = A_STEP + B_STEP;
    static constexpr int STAGES = (Q6 && NC == 256) ? 3 : 4;      // <= 4: one mins slot is enough (see the loader)
    static constexpr int SMEM = STAGES * STAGE + AM_BYTES + BM_BYTES + 1024;   // Q4_K: 148480 / 222208; Q6_K: 197632 / 197632
    // kind::f16 instruction descriptor: f32 accumulator, f16 x f16, both operands K-major, N = NC, M = 128
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NC >> 3) << 17) | ((uint32_t)(FQ_ROWS >> 4) << 24);
};

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
// two f32 fused multiply-adds in one instruction
__device__ __forceinline__ float2 q_fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(*reinterpret_cast<unsigned long long *>(&d)) : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)), "l"(*reinterpret_cast<unsigned long long *>(&c)));
    return d;
}
__device__ __forceinline__ void q_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem), "l"(adesc), "l"(bdesc),
                 "r"(idesc), "r"(accumulate)
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
// [7] producer warp 12 waiting for a free stage, [8] fetching ahead, [9] converting and storing, [10] proxy fence and arrival;
// [12] the CTA's whole run
__device__ unsigned long long g_fq_prof[16];
#define FQ_MARK(k)                                            \
    do {                                                      \
        if (prof) {                                           \
            const long long t_now = clock64();                \
            pacc[k] += (unsigned long long)(t_now - t_prev);  \
            t_prev = t_now;                                   \
        }                                                     \
    } while (0)

template <int NC, bool Q6>
struct alignas(16) FqBars {
    uint64_t full[FqCfg<NC, Q6>::STAGES], empty[FqCfg<NC, Q6>::STAGES], tfull[FQ_TSTAGES], tempty[FQ_TSTAGES];
    float da[FQ_DA_SLOTS][NC];
    uint32_t tmem_base;
    int abort_flag;
    int seen;   // the epilogue's verdict on a partial tile's flag, for all its warps
};

// up to three weight matrices of one type and row length against the same activations in one launch (the q / k / v
// projections of an attention block, the gate / up projections of an FFN): row block rb belongs to the last matrix e with
// rb_start[e] <= rb
struct FqMats {
    const uint8_t *tiles[3];
    float *dst[3];
    int64_t n[3], lddst[3];
    int rb_start[3];
    int count;
};

// a row's super-block takes the CUDA-core path for its mins: d == 0, or rho m_j could leave the f16 range
__device__ __forceinline__ bool q_mins_apart(float d, float dmin) { return !(fabsf(dmin) <= FQ_RHO_MAX * d); }

}  // namespace

// Q8_K activations of one block of NC rows and one super-block -> its B and Bm images and the scales.
template <int NC, bool Q6>
__global__ void __launch_bounds__(FQ_EXPAND_THREADS) expand_q8_K_acts_fast_kernel(ActView acts, uint8_t *bimg, int64_t m, int nb) {
    using C = FqCfg<NC, Q6>;
    pdl_trigger();
    pdl_wait();   // the activations come from the previous kernel, and the previous mat-mul may still be reading the images
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int b = blockIdx.x >> 2, g = blockIdx.x & 3;   // a CTA per (super-block, step): the launch is latency, not bytes
    const int64_t cb = blockIdx.y, K = acts.k;
    uint8_t *img = bimg + (cb * nb + b) * (int64_t)C::BIMG;
    // a warp reads 64 contiguous bytes (one pair) of 8 activation rows; piece r of the pair: (low p0, low p1, high p0,
    // high p1) -> chunks 4 p + 2 hi + {0, 1}
    const int r = lane >> 3, c0 = Q6 ? 2 * r : 4 * (r & 1) + 2 * (r >> 1);
#pragma unroll
    for (int rr = 0; rr < NC / 128; rr++) {
        const int bc = rr * 128 + warp * 8 + (lane & 7), sw = bc & 7;
        const int64_t col = cb * NC + bc;
        uint8_t *rowp = img + bc * 128;
        {
            uint4 y = make_uint4(0, 0, 0, 0);
            // Q4_K: step g = pair g, piece r of its 64 bytes.  Q6_K: step g = (n, l16) = (g / 2, g % 2), piece r = run r
            const int src_off = Q6 ? 128 * (g >> 1) + 32 * r + 16 * (g & 1) : g * 64 + r * 16;
            if (col < m) y = *(const uint4 *)(acts.qs + col * K + (int64_t)b * 256 + src_off);
            // a row past the end holds zeros: 0x80 after the flip, 128 - 128 = 0
            const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
            uint8_t *dstp = rowp + g * C::B_STEP;
            q_stg128(dstp + (((c0 + 0) ^ sw) << 4), q_signed(u0, 0), q_signed(u0, 8), q_signed(u1, 0), q_signed(u1, 8));
            q_stg128(dstp + (((c0 + 1) ^ sw) << 4), q_signed(u2, 0), q_signed(u2, 8), q_signed(u3, 0), q_signed(u3, 8));
        }
    }
    if (g != 0) return;   // the step-0 CTA also writes the super-block's sums and scales
    for (int i = tid; i < (Q6 ? 0 : 2 * NC); i += FQ_EXPAND_THREADS) {
        // sums: (row i / 2, half i % 2): eight 16-element sums -> one core-matrix row, written twice (K slots 0..15, 16..31)
        const int scol_i = i >> 1, kc = i & 1;
        const int64_t scol = cb * NC + scol_i;
        short4 b0 = make_short4(0, 0, 0, 0), b1 = b0;
        if (scol < m) {
            const short4 *bp = (const short4 *)(acts.bsums + scol * (K / 16) + (int64_t)b * 16 + 8 * kc);
            b0 = bp[0];
            b1 = bp[1];
        }
        uint8_t *bm = img + 4 * C::B_STEP + (scol_i >> 3) * 512 + (scol_i & 7) * 16 + kc * 128;
        const uint32_t v0 = q_h2_bits(__halves2half2(__short2half_rn(b0.x), __short2half_rn(b0.y))), v1 = q_h2_bits(__halves2half2(__short2half_rn(b0.z), __short2half_rn(b0.w)));
        const uint32_t v2 = q_h2_bits(__halves2half2(__short2half_rn(b1.x), __short2half_rn(b1.y))), v3 = q_h2_bits(__halves2half2(__short2half_rn(b1.z), __short2half_rn(b1.w)));
        q_stg128(bm, v0, v1, v2, v3);
        q_stg128(bm + 256, v0, v1, v2, v3);
    }
    for (int i = tid; i < NC; i += FQ_EXPAND_THREADS) {
        const int64_t dcol = cb * NC + i;
        reinterpret_cast<float *>(img + 4 * C::B_STEP + C::BM_BYTES)[i] = dcol < m ? acts.d[dcol * nb + b] : 0.0f;
    }
}

// Work split.  The mat-mul's work is the list of (output tile, super-block) units, tiles in (row block, column block) order
// with the column blocks of a row block adjacent; CTA p of P (at most one per SM) takes units U p / P .. U (p + 1) / P - 1, a
// contiguous run that may begin and end inside a tile.  A run's segment that covers a whole tile stores it.  A segment that
// begins inside a tile (it can only be the run's first, so it is done early) leaves its partial tile in the CTA's slot of
// a workspace and raises the CTA's flag; the segment that holds a tile's first super-block but not its last (it can only
// be the run's last) waits, bounded, for the flags of the CTAs after it that hold the tile's other parts, adds their
// partial tiles in ascending CTA order and stores: every output is summed in one fixed order whatever the timing.  The
// flags are lowered again by their reader.  Nobody waits for a CTA that waits, and every CTA is resident (the grid is at
// most one CTA per SM and a CTA takes an SM's whole shared memory or register file).
struct FqSplit {
    float *ws;          // [P][NC columns][128 rows] partial tiles
    unsigned *flags;    // [P]
    int gx;             // column blocks
    int total_tiles;
    unsigned wait_limit;   // polls of a partial tile's flag before the CTA gives up
    int mute_cta;          // test hook: this CTA leaves its flag down (-1: none)
};

template <int NC, bool Q6>
__global__ void __launch_bounds__(FQ_THREADS, 1)
gemm_kq_tcgen05_fast_kernel(const __grid_constant__ FqMats mats, const uint8_t *__restrict__ bimg, ActView acts, int nb, int64_t m, FqSplit sp, int *err,
                            int profile) {
    using C = FqCfg<NC, Q6>;
    constexpr int S = C::STAGES, CPT = NC / 2;   // columns per epilogue thread
    constexpr int CHUNK = Q6 ? 6720 : 4608;      // bytes of a 32-row tile's super-block
    extern __shared__ uint8_t fq_raw[];
    __shared__ FqBars<NC, Q6> bars;
    pdl_trigger();
    const uint32_t smem = (q_smem_u32(fq_raw) + 1023u) & ~1023u;
    const uint32_t mslot = smem + (uint32_t)(S * C::STAGE);   // Am | Bm of the super-block whose MMAs run
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int P = (int)gridDim.x, pcta = (int)blockIdx.x;
    const int64_t U = (int64_t)sp.total_tiles * nb;
    const int64_t u0 = U * pcta / P, u1 = U * (pcta + 1) / P;
    const int n_sb = (int)(u1 - u0);   // super-blocks of this CTA's run
    const int np = 4 * n_sb;           // pipeline steps: sub-block pairs
    volatile int *abort_flag = &bars.abort_flag;
    const bool prof = profile && blockIdx.x == 0 && lane == 0;
    long long t_prev = clock64();
    const long long t_start = t_prev;
    unsigned long long pacc[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};   // kept in registers, written once at the end
    // unit u -> its tile's matrix, row block within it and column block, and the super-block
    struct Unit {
        int mat, b;
        int64_t tile, rb, cb;
    };
    const auto unit_of = [&](int64_t u) {
        Unit x;
        x.tile = u / nb;
        x.b = (int)(u - x.tile * nb);
        const int64_t rbg = x.tile / sp.gx;
        x.cb = x.tile - rbg * sp.gx;
        x.mat = (mats.count > 2 && rbg >= mats.rb_start[2]) ? 2 : (mats.count > 1 && rbg >= mats.rb_start[1]) ? 1 : 0;
        x.rb = rbg - mats.rb_start[x.mat];
        return x;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < S; i++) {
            q_mbar_init(q_smem_u32(&bars.full[i]), 1 + FQ_PROD_WARPS);   // the loader's arrive + the bytes it announced + the producer warps
            q_mbar_init(q_smem_u32(&bars.empty[i]), 1);                  // the MMA thread's commit
        }
        for (int i = 0; i < FQ_TSTAGES; i++) {
            q_mbar_init(q_smem_u32(&bars.tfull[i]), 1);
            q_mbar_init(q_smem_u32(&bars.tempty[i]), FQ_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == FQ_MMA_WARP) {
        // both tensor-memory stages; the CTA's shared memory (or, with 128 columns, its registers) keeps a second CTA off this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(q_smem_u32(&bars.tmem_base)), "r"(FQ_TSTAGES * NC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;

    if (warp < FQ_EPI_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(FQ_REGS_EPI));
        pdl_wait();   // the previous kernels in the stream may still read dst
        const int q = warp & 3, h = warp >> 2;
        const uint32_t trow0 = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(CPT * h);
        float *my_ws = sp.ws + ((size_t)pcta * NC + CPT * h) * FQ_ROWS + 32 * q + lane;   // + column * 128
        float2 acc[CPT / 2];
        bool ok = true;
        int jb = 0;   // super-blocks of the run done so far: tensor-memory stage and scale slot
        while (jb < n_sb && ok) {
            // ---- one segment: super-blocks b_first .. b_last of one tile
            const Unit un = unit_of(u0 + jb);
            const int b_first = un.b, seg = (nb - b_first) < (n_sb - jb) ? (nb - b_first) : (n_sb - jb), b_last = b_first + seg - 1;
            const uint8_t *tiles = mats.tiles[un.mat];
            float *dst = mats.dst[un.mat];
            const int64_t n = mats.n[un.mat], lddst = mats.lddst[un.mat];
            const int64_t tile0 = un.rb * (FQ_ROWS / TILE_ROWS), tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS, col0 = un.cb * NC;
            const bool row_ok = tile0 + q < tiles_n;
            const bool any_col = col0 + CPT * h < m;
            // (d, dmin) of this thread's row (Q6_K: d), one word per super-block, fetched one super-block ahead
            const uint8_t *hdr = tiles + (row_ok ? tile0 + q : 0) * (int64_t)nb * CHUNK + (Q6 ? 6656 + lane * 2 : lane * 16);
            const auto load_dd = [&](int b) -> uint32_t { return Q6 ? (uint32_t) * (const uint16_t *)(hdr + (int64_t)b * CHUNK) : *(const uint32_t *)(hdr + (int64_t)b * CHUNK); };
            uint32_t dd_next = row_ok ? load_dd(b_first) : 0u;
#pragma unroll
            for (int c = 0; c < CPT / 2; c++) acc[c] = make_float2(0.0f, 0.0f);
            bool any_apart = false;
            for (int b = b_first; b <= b_last; b++, jb++) {
                const int t = jb % FQ_TSTAGES;
                const float dw = f16_bits_to_f32((uint16_t)(dd_next & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(dd_next >> 16));
                any_apart |= !Q6 && row_ok && dmw != 0.0f && q_mins_apart(dw, dmw);
                if (b < b_last && row_ok) dd_next = load_dd(b + 1);
                if (warp == 0) FQ_MARK(1);
                if (!__all_sync(0xffffffffu, q_mbar_wait(q_smem_u32(&bars.tfull[t]), (uint32_t)(jb / FQ_TSTAGES) & 1u, abort_flag))) {
                    ok = false;
                    break;
                }
                if (warp == 0) FQ_MARK(0);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float4 *das = reinterpret_cast<const float4 *>(bars.da[jb % FQ_DA_SLOTS] + CPT * h);
                const uint32_t trow = trow0 + (uint32_t)(t * NC);
                const float2 dw2 = make_float2(dw, dw), zero2 = make_float2(0.0f, 0.0f);
                // rounds of 32 columns, one tensor-memory round trip each: acc += (d_x d) v, two columns per instruction
                uint32_t v[32];
#pragma unroll
                for (int r = 0; r < CPT / 32; r++) {
                    q_tmem_ld32(v, trow + (uint32_t)(32 * r));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (r == CPT / 32 - 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.tempty[t]));
                    }
                    if (any_col) {
#pragma unroll
                        for (int c4 = 0; c4 < 8; c4++) {
                            const float4 dq = das[8 * r + c4];
                            const float2 s0 = q_fma2(make_float2(dq.x, dq.y), dw2, zero2), s1 = q_fma2(make_float2(dq.z, dq.w), dw2, zero2);
                            acc[16 * r + 2 * c4] = q_fma2(make_float2(__uint_as_float(v[4 * c4]), __uint_as_float(v[4 * c4 + 1])), s0, acc[16 * r + 2 * c4]);
                            acc[16 * r + 2 * c4 + 1] = q_fma2(make_float2(__uint_as_float(v[4 * c4 + 2]), __uint_as_float(v[4 * c4 + 3])), s1, acc[16 * r + 2 * c4 + 1]);
                        }
                    }
                }
            }
            if (!ok) break;
            // ---- the segment's outputs
            const int64_t row = (tile0 + q) * TILE_ROWS + lane;
            const bool partial = b_first > 0;   // begun by an earlier CTA: this one's part goes to the workspace
            // the super-blocks whose mins the tensor core did not take: -= d_x dmin sum_j m_j (bsum_2j + bsum_2j+1), applied to
            // what this thread has just stored (its row of the tile, or of the partial tile)
            const auto mins_apart = [&]() {
                if constexpr (!Q6) {
                    if (!(any_apart && row_ok && row < n)) return;
                    for (int b = b_first; b <= b_last; b++) {
                        const uint4 hd = *(const uint4 *)(tiles + ((tile0 + q) * (int64_t)nb + b) * CHUNK + lane * 16);
                        const float dw = f16_bits_to_f32((uint16_t)(hd.x & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(hd.x >> 16));
                        if (dmw == 0.0f || !q_mins_apart(dw, dmw)) continue;
                        const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
                        for (int c = 0; c < CPT; c++) {
                            const int64_t col = col0 + CPT * h + c;
                            if (col >= m) break;
                            const int16_t *bs = acts.bsums + col * (acts.k / 16) + (int64_t)b * 16;
                            int mg = 0;
                            for (int j = 0; j < 8; j++) mg += (int)(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu) * ((int)bs[2 * j] + (int)bs[2 * j + 1]);
                            const float sub = acts.d[col * nb + b] * dmw * (float)mg;
                            if (partial) my_ws[(size_t)c * FQ_ROWS] -= sub;
                            else dst[col * lddst + row] -= sub;
                        }
                    }
                }
            };
            if (partial) {
#pragma unroll
                for (int c = 0; c < CPT; c++) my_ws[(size_t)c * FQ_ROWS] = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                mins_apart();
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(FQ_EPI_WARPS * 32) : "memory");
                if (threadIdx.x == 0 && pcta != sp.mute_cta) atomicExch(sp.flags + pcta, 1u);
                continue;
            }
            if (b_last < nb - 1) {
                // the tile's first super-blocks, the rest is with the CTAs after this one: their partial tiles, in ascending order
                int qhi = pcta + 1;
                while (qhi < P - 1 && U * (qhi + 1) / P < (un.tile + 1) * nb) qhi++;   // the CTA whose run holds the tile's last super-block
                for (int qq = pcta + 1; qq <= qhi; qq++) {
                    if (threadIdx.x == 0) {
                        bool seen = false;
                        for (uint32_t itw = 0; itw < sp.wait_limit && !seen; itw++) {
                            seen = *(volatile unsigned *)(sp.flags + qq) != 0u;
                            if (!seen && (itw & 255) == 255 && *abort_flag) break;
                        }
                        if (!seen) *abort_flag = 1;
                        bars.seen = seen ? 1 : 0;
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(FQ_EPI_WARPS * 32) : "memory");
                    if (!*(volatile int *)&bars.seen) {
                        ok = false;
                        break;
                    }
                    __threadfence();
                    const float *ows = sp.ws + ((size_t)qq * NC + CPT * h) * FQ_ROWS + 32 * q + lane;
#pragma unroll
                    for (int c = 0; c < CPT; c += 2) {
                        acc[c >> 1].x = __fadd_rn(acc[c >> 1].x, __ldcg(ows + (size_t)c * FQ_ROWS));
                        acc[c >> 1].y = __fadd_rn(acc[c >> 1].y, __ldcg(ows + (size_t)(c + 1) * FQ_ROWS));
                    }
                    // every epilogue warp has read the slot: its flag goes down for the next launch
                    asm volatile("bar.sync 1, %0;" ::"n"(FQ_EPI_WARPS * 32) : "memory");
                    if (threadIdx.x == 0) atomicExch(sp.flags + qq, 0u);
                }
                if (!ok) break;
            }
            if (row_ok && row < n) {
#pragma unroll
                for (int c = 0; c < CPT; c++) {
                    const int64_t col = col0 + CPT * h + c;
                    if (col < m) dst[col * lddst + row] = (c & 1) ? acc[c >> 1].y : acc[c >> 1].x;
                }
            }
            mins_apart();
        }
    } else if (warp >= FQ_PROD_WARP0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FQ_REGS_PROD));
        const int tt = warp - FQ_PROD_WARP0, prow = tt * 32 + lane, sw = prow & 7;
        uint8_t *stage0 = fq_raw + (smem - q_smem_u32(fq_raw)) + prow * 128;
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        // the row's bytes of super-block unit u0 + js (nullptr past the matrix's last row tile or the run's end)
        const auto chunk_of = [&](int js) -> const uint8_t * {
            if (js >= n_sb) return nullptr;
            const Unit un = unit_of(u0 + js);
            const int64_t tile = un.rb * (FQ_ROWS / TILE_ROWS) + tt;
            if (tile >= (mats.n[un.mat] + TILE_ROWS - 1) / TILE_ROWS) return nullptr;
            return mats.tiles[un.mat] + (tile * (int64_t)nb + un.b) * CHUNK + lane * 16;
        };
        if constexpr (Q6) {
            // thread = row (tile tt, lane): per step (n, l16) = (g / 2, g % 2) the 16-byte pieces ql[4 n + l16], ql[4 n + 2 + l16] and
            // qh[2 n + l16] of its super-block, loaded two steps ahead (the weights do not depend on the previous kernel)
            uint4 sc = zero4, sc_next = zero4, w[4][3];
#pragma unroll
            for (int i = 0; i < 4; i++) w[i][0] = w[i][1] = w[i][2] = zero4;
            const auto fetch = [&](const uint8_t *c, int g, uint4(&dst3)[3]) {
                const int n = g >> 1, l16 = g & 1;
                if (c) {
                    dst3[0] = ld_stream16(c + (4 * n + l16) * 512);
                    dst3[1] = ld_stream16(c + (4 * n + 2 + l16) * 512);
                    dst3[2] = ld_stream16(c + 4096 + (2 * n + l16) * 512);
                } else {
                    dst3[0] = dst3[1] = dst3[2] = zero4;
                }
            };
            const uint8_t *cur = chunk_of(0), *nxt = chunk_of(1);
            if (cur) sc_next = *(const uint4 *)(cur + 6144);
            if (n_sb > 0) {
                fetch(cur, 0, w[0]);
                fetch(cur, 1, w[1]);
            }
            bool ok = true;
            for (int js = 0; js < n_sb && ok; js++) {
                sc = sc_next;
                sc_next = nxt ? *(const uint4 *)(nxt + 6144) : zero4;
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const int p = 4 * js + g, s = p % S;
                    if (g < 2) fetch(cur, g + 2, w[g + 2]);   // set (g + 2) % 4 was consumed two steps ago
                    else fetch(nxt, g - 2, w[g - 2]);
                    if (warp == FQ_PROD_WARP0) FQ_MARK(8);
                    if (!__all_sync(0xffffffffu, q_mbar_wait(q_smem_u32(&bars.empty[s]), ((uint32_t)(p / S) & 1u) ^ 1u, abort_flag))) {
                        ok = false;
                        break;
                    }
                    if (warp == FQ_PROD_WARP0) FQ_MARK(7);
                    uint8_t *hip = stage0 + s * C::STAGE, *lop = hip + FQ_A_STEP;
                    const uint4 A = w[g][0], B = w[g][1], H = w[g][2];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        // run r: elements 128 n + 32 r + 16 l16 .. + 15, scale 8 n + 2 r + l16
                        const int si = 8 * (g >> 1) + 2 * r + (g & 1);
                        const uint32_t sword = si < 4 ? sc.x : si < 8 ? sc.y : si < 12 ? sc.z : sc.w;
                        const __half sh = __int2half_rn((int)(int8_t)(sword >> (8 * (si & 3))));
                        const __half2 s2 = __halves2half2(sh, sh);
                        const __half2 chi = __hmul2(s2, __float2half2_rn(-96.0f)), clo = __hmul2(s2, __float2half2_rn(-64.0f));
                        uint32_t hi[8], lo[8];
#pragma unroll
                        for (int wd = 0; wd < 4; wd++) {
                            const uint32_t aw = wd == 0 ? A.x : wd == 1 ? A.y : wd == 2 ? A.z : A.w, bw = wd == 0 ? B.x : wd == 1 ? B.y : wd == 2 ? B.z : B.w;
                            const uint32_t hw = wd == 0 ? H.x : wd == 1 ? H.y : wd == 2 ? H.z : H.w;
                            const uint32_t v = r == 0   ? (aw & 0x0f0f0f0fu) | ((hw << 4) & 0x30303030u)
                                               : r == 1 ? (bw & 0x0f0f0f0fu) | ((hw << 2) & 0x30303030u)
                                               : r == 2 ? ((aw >> 4) & 0x0f0f0f0fu) | (hw & 0x30303030u)
                                                        : ((bw >> 4) & 0x0f0f0f0fu) | ((hw >> 2) & 0x30303030u);
                            const uint32_t v8 = v >> 8;
                            // (64 + 8 (q >> 3)) s - 96 s = s (8 (q >> 3) - 32);  (64 + (q & 7)) s - 64 s = s (q & 7): one rounding each, exact
                            hi[2 * wd] = q_h2_bits(__hfma2(q_bits_h2(((v & 0x00380038u) << 4) | 0x54005400u), s2, chi));
                            hi[2 * wd + 1] = q_h2_bits(__hfma2(q_bits_h2(((v8 & 0x00380038u) << 4) | 0x54005400u), s2, chi));
                            lo[2 * wd] = q_h2_bits(__hfma2(q_bits_h2(((v & 0x00070007u) << 4) | 0x54005400u), s2, clo));
                            lo[2 * wd + 1] = q_h2_bits(__hfma2(q_bits_h2(((v8 & 0x00070007u) << 4) | 0x54005400u), s2, clo));
                        }
                        q_stg128(hip + (((2 * r + 0) ^ sw) << 4), hi[0], hi[1], hi[2], hi[3]);
                        q_stg128(hip + (((2 * r + 1) ^ sw) << 4), hi[4], hi[5], hi[6], hi[7]);
                        q_stg128(lop + (((2 * r + 0) ^ sw) << 4), lo[0], lo[1], lo[2], lo[3]);
                        q_stg128(lop + (((2 * r + 1) ^ sw) << 4), lo[4], lo[5], lo[6], lo[7]);
                    }
                    if (warp == FQ_PROD_WARP0) FQ_MARK(9);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.full[s]));
                    if (warp == FQ_PROD_WARP0) FQ_MARK(10);
                }
                cur = nxt;
                nxt = chunk_of(js + 2);
            }
        } else {
            // thread = row (tile tt, lane): per step the two 16-byte pieces 2 g, 2 g + 1 of its 128 nibble bytes, loaded three steps
            // ahead into register set (step + 3) % 4 (the weights do not depend on the previous kernel)
            uint8_t *am = fq_raw + (mslot - q_smem_u32(fq_raw)) + (prow >> 3) * 512 + (prow & 7) * 16;
            uint4 hd = zero4, hd_next = zero4, w[4][2];
#pragma unroll
            for (int i = 0; i < 4; i++) w[i][0] = w[i][1] = zero4;
            const auto fetch = [&](const uint8_t *c, int g, uint4(&dst2)[2]) {
                if (c) {
                    dst2[0] = ld_stream16(c + 512 + (2 * g) * 512);
                    dst2[1] = ld_stream16(c + 512 + (2 * g + 1) * 512);
                } else {
                    dst2[0] = dst2[1] = zero4;
                }
            };
            const uint8_t *cur = chunk_of(0), *nxt = chunk_of(1);
            if (cur) hd_next = *(const uint4 *)cur;
            if (n_sb > 0) {
                fetch(cur, 0, w[0]);
                fetch(cur, 1, w[1]);
                fetch(cur, 2, w[2]);
            }
            bool ok = true;
            for (int js = 0; js < n_sb && ok; js++) {
                hd = hd_next;
                hd_next = nxt ? *(const uint4 *)nxt : zero4;
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const int p = 4 * js + g, s = p % S;
                    if (g == 0) fetch(cur, 3, w[3]);   // set (g + 3) % 4 was consumed in the previous step
                    else fetch(nxt, g - 1, w[g - 1]);
                    if (warp == FQ_PROD_WARP0) FQ_MARK(8);
                    if (!__all_sync(0xffffffffu, q_mbar_wait(q_smem_u32(&bars.empty[s]), ((uint32_t)(p / S) & 1u) ^ 1u, abort_flag))) {
                        ok = false;
                        break;
                    }
                    if (warp == FQ_PROD_WARP0) FQ_MARK(7);
                    if (g == 0) {
                        // the mins slot is free: the stage this step reuses was released by MMAs issued after those of the previous
                        // super-block's first step.  -rho m_j as high part + remainder; all zero where the drain takes the mins
                        const float dw = f16_bits_to_f32((uint16_t)(hd.x & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(hd.x >> 16));
                        const float nrho = (dmw == 0.0f || q_mins_apart(dw, dmw)) ? 0.0f : -(dmw / dw);
                        const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
                        uint32_t hi[8], lo[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float v = nrho * (float)(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xffu);
                            const __half vh = __float2half_rn(v);
                            const __half vl = __float2half_rn(v - __half2float(vh));
                            hi[j] = q_h2_bits(__halves2half2(vh, vh));
                            lo[j] = q_h2_bits(__halves2half2(vl, vl));
                        }
                        q_stg128(am, hi[0], hi[1], hi[2], hi[3]);
                        q_stg128(am + 128, hi[4], hi[5], hi[6], hi[7]);
                        q_stg128(am + 256, lo[0], lo[1], lo[2], lo[3]);
                        q_stg128(am + 384, lo[4], lo[5], lo[6], lo[7]);
                    }
                    {
                        // pair g: sub-blocks 2 g, 2 g + 1
                        const uint32_t scw = g < 2 ? (hd.y & 0x3f3f3f3fu) : ((hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
                        const uint32_t s_lo = (scw >> (16 * (g & 1))) & 0xffu, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xffu;
                        const __half2 sl = q_small2(s_lo), sh = q_small2(s_hi);
                        // -1024 s <= 64512 in magnitude: a multiple of 1024 below 65504, exact in f16
                        const __half2 cl = __hmul2(sl, __float2half2_rn(-1024.0f)), ch = __hmul2(sh, __float2half2_rn(-64.0f));
                        const __half2 sh16 = __hmul2(sh, __float2half2_rn(0.0625f));
                        uint8_t *dstp = stage0 + s * C::STAGE;
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const uint4 x = w[g][i];
                            const uint32_t x8 = x.x >> 8, y8 = x.y >> 8, z8 = x.z >> 8, w8 = x.w >> 8;   // bytes 1 and 3
                            const int c0 = 4 * i;
                            q_stg128(dstp + (((c0 + 0) ^ sw) << 4), q_scaled_lo(x.x, sl, cl), q_scaled_lo(x8, sl, cl), q_scaled_lo(x.y, sl, cl), q_scaled_lo(y8, sl, cl));
                            q_stg128(dstp + (((c0 + 1) ^ sw) << 4), q_scaled_lo(x.z, sl, cl), q_scaled_lo(z8, sl, cl), q_scaled_lo(x.w, sl, cl), q_scaled_lo(w8, sl, cl));
                            q_stg128(dstp + (((c0 + 2) ^ sw) << 4), q_scaled_hi(x.x, sh16, ch), q_scaled_hi(x8, sh16, ch), q_scaled_hi(x.y, sh16, ch), q_scaled_hi(y8, sh16, ch));
                            q_stg128(dstp + (((c0 + 3) ^ sw) << 4), q_scaled_hi(x.z, sh16, ch), q_scaled_hi(z8, sh16, ch), q_scaled_hi(x.w, sh16, ch), q_scaled_hi(w8, sh16, ch));
                        }
                    }
                    if (warp == FQ_PROD_WARP0) FQ_MARK(9);
                    // the stores (generic proxy) before the tensor core's reads (async proxy), then the warp's arrival
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) q_mbar_arrive(q_smem_u32(&bars.full[s]));
                    if (warp == FQ_PROD_WARP0) FQ_MARK(10);
                }
                cur = nxt;
                nxt = chunk_of(js + 2);
            }
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(FQ_REGS_CTL));
        pdl_wait();   // the images are the previous kernel's output
        if (warp == FQ_MMA_WARP) {
            if (lane == 0) {
                for (int p = 0; p < np; p++) {
                    const int s = p % S, jb = p >> 2, g = p & 3, t = jb % FQ_TSTAGES;
                    FQ_MARK(4);
                    if (!q_mbar_wait(q_smem_u32(&bars.full[s]), (uint32_t)(p / S) & 1u, abort_flag)) break;
                    FQ_MARK(2);
                    if (g == 0 && !q_mbar_wait(q_smem_u32(&bars.tempty[t]), ((uint32_t)(jb / FQ_TSTAGES) & 1u) ^ 1u, abort_flag)) break;
                    FQ_MARK(3);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_base = smem + (uint32_t)(s * C::STAGE), b_base = a_base + C::A_STEP;
                    const uint32_t d_acc = tmem + (uint32_t)(t * NC);
                    const uint64_t ad = q_desc_sw128(a_base), bd = q_desc_sw128(b_base);
                    if constexpr (Q6) {
                        const uint64_t ad_lo = q_desc_sw128(a_base + FQ_A_STEP);
#pragma unroll
                        for (int i = 0; i < 4; i++) {   // K = 16 step i: 32 bytes on; the high parts, then the low parts, of the same 16 elements
                            q_mma(d_acc, ad + 2 * i, bd + 2 * i, C::IDESC, (g | i) != 0);
                            q_mma(d_acc, ad_lo + 2 * i, bd + 2 * i, C::IDESC, 1);
                        }
                    } else {
                        if (g == 0) {
                            // the mins first (they clear the accumulator): K = 32 as two MMAs, core-matrix columns 0, 1 and 2, 3
                            const uint64_t amd = q_desc_plain(mslot, 128, 512), bmd = q_desc_plain(mslot + FQ_AM_BYTES, 128, 512);
                            q_mma(d_acc, amd, bmd, C::IDESC, 0);
                            q_mma(d_acc, amd + (256 >> 4), bmd + (256 >> 4), C::IDESC, 1);
                        }
#pragma unroll
                        for (int i = 0; i < 4; i++) q_mma(d_acc, ad + 2 * i, bd + 2 * i, C::IDESC, 1);   // K = 16 step i: 32 bytes on
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(q_smem_u32(&bars.empty[s])) : "memory");
                    if (g == 3)
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(q_smem_u32(&bars.tfull[t])) : "memory");
                }
            }
        } else if (warp == FQ_LOAD_WARP && lane == 0) {
            int issued = -1;
            const uint8_t *bb = nullptr;
            for (int p = 0; p < np; p++) {
                const int s = p % S, jb = p >> 2, g = p & 3;
                if (g == 0) {
                    const Unit un = unit_of(u0 + jb);
                    bb = bimg + (un.cb * nb + un.b) * (int64_t)C::BIMG;
                }
                FQ_MARK(6);
                if (!q_mbar_wait(q_smem_u32(&bars.empty[s]), ((uint32_t)(p / S) & 1u) ^ 1u, abort_flag)) break;
                FQ_MARK(5);
                const uint32_t bar = q_smem_u32(&bars.full[s]), stage = smem + (uint32_t)(s * C::STAGE);
                q_mbar_expect(bar, (uint32_t)(C::B_STEP + (g == 0 ? C::BM_BYTES + C::DA_BYTES : 0)));
                q_bulk_load(stage + C::A_STEP, bb + g * C::B_STEP, C::B_STEP, bar);
                if (g == 0) {
                    // the mins slot: with at most four stages the stage this step reuses belonged to a step of the previous
                    // super-block no earlier than its first, so that super-block's mins MMAs are done; the scale slot of
                    // super-block jb - 4: its drain ended before the MMAs of jb - 2 began
                    if constexpr (!Q6) q_bulk_load(mslot + FQ_AM_BYTES, bb + 4 * C::B_STEP, C::BM_BYTES, bar);
                    q_bulk_load(q_smem_u32(bars.da[jb % FQ_DA_SLOTS]), bb + 4 * C::B_STEP + C::BM_BYTES, C::DA_BYTES, bar);
                }
                issued = p;
            }
            // a CTA that gives up still waits (bounded) for the copies it has in flight
            if (*abort_flag && issued >= 0) q_mbar_wait(q_smem_u32(&bars.full[issued % S]), (uint32_t)(issued / S) & 1u, abort_flag);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == FQ_MMA_WARP) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(FQ_TSTAGES * NC) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, FQ_ERR_WAIT);
    if (prof) {
#pragma unroll
        for (int i = 0; i < 12; i++)
            if (pacc[i]) atomicAdd(&g_fq_prof[i], pacc[i]);
        if (threadIdx.x == 0) atomicAdd(&g_fq_prof[12], (unsigned long long)(clock64() - t_start));
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

// flags of the partial tiles: one word per CTA of the grid, all zero between launches (a module variable: no allocation)
__device__ unsigned g_fq_flags[1024];

// test hook: while spin_limit > 0 the wait for a partial tile's flag polls at most spin_limit times and CTA mute_cta never
// raises its flag, so that a test can watch that wait run out (the kernel returns, error code 4)
static int g_fq_wait_limit_override = 0, g_fq_mute_cta = -1;
void gemm_fast_debug_wait(int spin_limit, int mute_cta) {
    g_fq_wait_limit_override = spin_limit > 0 ? spin_limit : 0;
    g_fq_mute_cta = mute_cta;
}

// after a launch that gave up (a bounded wait ran out) flags may be left raised: lower them all, after the device has drained
int gemm_fast_reset_flags() {
    B200_CUDA(cudaDeviceSynchronize());
    static const unsigned zeros[1024] = {0};
    B200_CUDA(cudaMemcpyToSymbol(g_fq_flags, zeros, sizeof(zeros)));
    return B200_STATUS_SUCCESS;
}

template <int NC, bool Q6>
static int launch_fast(const FqMats &mats, int64_t gy, int64_t k, int64_t m, ActView acts, int *err, int profile, int sms, cudaStream_t s) {
    using C = FqCfg<NC, Q6>;
    static bool attr_done[64] = {false};
    static unsigned *flags[64] = {nullptr};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_kq_tcgen05_fast_kernel<NC, Q6>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        void *fp = nullptr;
        B200_CUDA(cudaGetSymbolAddress(&fp, g_fq_flags));
        flags[dev] = (unsigned *)fp;
        attr_done[dev] = true;
    }
    const int nb = (int)(k / GROUP_K);
    const int64_t gx = (m + NC - 1) / NC;
    B200_REQUIRE(gx <= 65535 && gy * gx < (1ll << 31) / nb, "gemm: %lld row blocks x %lld column blocks are too many for one launch", (long long)gy, (long long)gx);
    // At most one CTA per SM, each a contiguous run of (tile, super-block) units.  How many: a run costs its super-blocks, plus,
    // where runs cut tiles, the partial tiles the tile's owner has to add one after the other (measured: about 0.85 of a
    // super-block's time each) and the write of its own (0.4).  1024 x 4096 x 512: 148 CTAs 56 us, 64 CTAs 38 us; 4096 x 4096 x
    // 512: 148 CTAs 46 us, 128 CTAs (every tile in two halves) 43 us.  B200_GEMM_FAST_CTAS=<n> sets the count (read per call;
    // the tests use it to cut tiles in odd places)
    const int64_t units = gy * gx * nb;
    int64_t ctas = 1;
    {
        double best = 1e300;
        const int64_t hi = units < sms ? units : sms;
        for (int64_t pc = hi; pc >= 1 && pc >= hi / 4; pc--) {
            const double run = (double)units / (double)pc;
            const int64_t run_up = (units + pc - 1) / pc;
            const bool whole = units % pc == 0 && (run_up % nb == 0 || nb % run_up == 0);   // every run ends where a tile or an even part of one ends
            const double pieces = run >= nb ? (whole && run_up % nb == 0 ? 1.0 : 2.0) : std::ceil((double)nb / run) + (whole ? 0.0 : 1.0);
            const double cost = (double)run_up + 0.85 * (pieces - 1.0) + (pieces > 1.0 ? 0.4 : 0.0);
            if (cost < best) {
                best = cost;
                ctas = pc;
            }
        }
    }
    if (const char *cv = getenv("B200_GEMM_FAST_CTAS")) {
        const long v = atol(cv);
        if (v >= 1 && v <= sms && v <= units) ctas = v;
    }
    B200_REQUIRE(ctas <= 1024, "gemm: %lld CTAs exceed the partial-tile flags", (long long)ctas);
    const size_t img_bytes = (size_t)gx * nb * C::BIMG, ws_bytes = (size_t)ctas * NC * FQ_ROWS * 4;
    void *block = nullptr;
    int rc = scratch_get_images(img_bytes + ws_bytes, &block);
    if (rc != B200_STATUS_SUCCESS) return rc;
    uint8_t *bimg = (uint8_t *)block;
    FqSplit sp;
    sp.ws = (float *)(bimg + img_bytes);
    sp.flags = flags[dev];
    sp.gx = (int)gx;
    sp.total_tiles = (int)(gy * gx);
    sp.wait_limit = g_fq_wait_limit_override > 0 ? (unsigned)g_fq_wait_limit_override : FQ_WAIT_LIMIT;
    sp.mute_cta = g_fq_wait_limit_override > 0 ? g_fq_mute_cta : -1;
    rc = launch_pdl(expand_q8_K_acts_fast_kernel<NC, Q6>, dim3((unsigned)(4 * nb), (unsigned)gx), dim3(FQ_EXPAND_THREADS), (size_t)0, s, acts, bimg, m, nb);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_pdl(gemm_kq_tcgen05_fast_kernel<NC, Q6>, dim3((unsigned)ctas), dim3(FQ_THREADS), (size_t)C::SMEM, s, mats, (const uint8_t *)bimg, acts, nb, m, sp,
                      err, profile);
}

// type: B200_TYPE_Q4_K or B200_TYPE_Q6_K; count matrices (1 .. 3) of that type and row length k over the same m activation rows
int launch_gemm_kq_fast_multi(int type, int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                              const int64_t *lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    B200_REQUIRE(type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K, "gemm: the fast kernel takes Q4_K and Q6_K, not type %d", type);
    B200_REQUIRE(count >= 1 && count <= 3, "gemm: %d matrices in one launch (1 .. 3)", count);
    if (m == 0) return B200_STATUS_SUCCESS;
    FqMats mats;
    memset(&mats, 0, sizeof(mats));
    int64_t gy = 0;
    for (int e = 0; e < count; e++) {
        if (n[e] == 0) continue;
        const int c = mats.count++;
        mats.tiles[c] = tiles[e];
        mats.dst[c] = dst[e];
        mats.n[c] = n[e];
        mats.lddst[c] = lddst[e];
        mats.rb_start[c] = (int)gy;
        gy += (n[e] + FQ_ROWS - 1) / FQ_ROWS;
    }
    if (mats.count == 0) return B200_STATUS_SUCCESS;
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const char *pv = getenv("B200_GEMM_FAST_PROFILE");
    const int profile = pv && pv[0] == '1';
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    // 256 activation rows per CTA run the tensor core at its rate (an M 128 x K 16 MMA takes 128 cycles whatever N <= 256 is):
    // taken whenever there are more than 128 rows.  B200_GEMM_FAST_COLS=128 / 256 overrides (read per call)
    bool wide = m > 128;
    if (const char *cv = getenv("B200_GEMM_FAST_COLS")) wide = cv[0] == '2' ? true : cv[0] == '1' ? false : wide;
    if (type == B200_TYPE_Q6_K)
        return wide ? launch_fast<256, true>(mats, gy, k, m, acts, err, profile, sms, s) : launch_fast<128, true>(mats, gy, k, m, acts, err, profile, sms, s);
    return wide ? launch_fast<256, false>(mats, gy, k, m, acts, err, profile, sms, s) : launch_fast<128, false>(mats, gy, k, m, acts, err, profile, sms, s);
}

int launch_gemm_kq_fast(int type, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    return launch_gemm_kq_fast_multi(type, 1, &n, k, m, &tiles, acts, &dst, &lddst, s);
}

int launch_gemm_q4_K_fast(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s) {
    return launch_gemm_kq_fast(B200_TYPE_Q4_K, n, k, m, tiles, acts, dst, lddst, s);
}

}  // namespace b200
