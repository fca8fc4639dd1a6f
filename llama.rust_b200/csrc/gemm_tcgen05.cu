// Prompt-shaped Q4_K mat-mul on the fifth-generation tensor cores: tcgen05.mma kind::i8 with the
// sub-block dots accumulated in tensor memory, fed from shared memory by producer warps that unpack the
// 4-bit weights to int8 on the way in, and drained by epilogue warps that run the CPU route's f32 chain.
//
// Arithmetic (identical to gemm_mma.cu, which computes the same dots with mma.sync): the CPU routes never add
// two sub-blocks' integer dots before scaling them, so one MMA (M 128 weight rows x N 32 activation rows x
// K 32) computes exactly one 32-element sub-block's dots, with the accumulator cleared, into its own 32
// tensor-memory columns; eight MMAs cover a 256-element super-block and fill one 256-column stage.  The
// epilogue thread that owns a weight row reads its dots back (tcgen05.ld), applies the 6-bit sub-block
// scales in integer arithmetic and feeds
//   8x8 gemm route (crates/ggml/src/repack.rs:1692-1768), per sub-block pair g:
//         sumf = fma(f32(ig[g]), d*d_x, sumf); summin = fma(f32(mg[g]), dmin*d_x, summin); out = sumf - summin
//   tiled route    (crates/ggml/src/tiled.rs:823-838), per super-block:
//         r = d*f32(s1); r = fma(-dmin, f32(s2), r); out = fma(r, d_x, out)
// so the result is bit-identical to the decode kernels' and to the CPU's.
//
// One CTA = 128 weight rows (four 32-row tiles of the device layout) x 32 activation rows, walking K one
// super-block per pipeline step:
//   warps 0-7   epilogue: warp w owns tensor-memory lanes 32 (w % 4) .. + 31 (weight rows) and activation
//               rows 16 (w / 4) .. + 15; 8 warps keep two chains per scheduler in flight
//   warps 8-11  producers: nibbles -> int8 into the A operand, int8 activation blocks into the B operand
//               (both K-major, no swizzle: 8 rows x 16 bytes core matrices, K-adjacent ones 128 bytes apart,
//               8-row groups 2048 bytes apart), pair sums of the activation bsums and the activation scales
//   warp 12     tensor-memory allocation and, one lane, the MMA issue + commits
// Shared memory holds three operand stages, tensor memory two accumulator stages; all hand-offs are
// mbarriers.  Every wait is bounded: a wait that runs out raises the CTA's abort flag and the device error
// word, every role leaves its loop, and the CTA frees its tensor memory and returns.
//
// The second kernel in this file (gemm_q4_K_tcgen05_f16_kernel, further down) folds the sub-block scales into
// f16 operands so that the MMA returns the chain's integers as f32 and the epilogue shrinks to two fmas.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int TC_ROWS = 128;                 // weight rows per CTA (MMA M)
constexpr int TC_COLS = 32;                  // activation rows per CTA (MMA N)
constexpr int TC_EPI_WARPS = 8, TC_PROD_WARPS = 4;
constexpr int TC_THREADS = (TC_EPI_WARPS + TC_PROD_WARPS + 1) * 32;
constexpr int TC_STAGES = 3;                 // shared-memory operand stages
constexpr int TC_TSTAGES = 2;                // tensor-memory accumulator stages of 8 * TC_COLS columns
constexpr int TC_A_BYTES = TC_ROWS * 256;    // one super-block of int8 weights
constexpr int TC_B_BYTES = TC_COLS * 256;
constexpr int TC_BP_BYTES = 4 * TC_COLS * 8; // [pair][column] (sum of low sub-block, sum of high sub-block)
constexpr int TC_DA_BYTES = TC_COLS * 4;
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES + TC_BP_BYTES + TC_DA_BYTES;
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;   // tries per wait before the CTA gives up
constexpr int TC_ERR_WAIT = 4;               // device error word: a pipeline wait ran out

// kind::i8 instruction descriptor: s32 accumulator, s8 x s8, both operands K-major, N = 32, M = 128
constexpr uint32_t TC_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_COLS >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor, no swizzle: start address, 128 bytes between K-adjacent core matrices
// (leading byte offset), 2048 bytes between 8-row groups (stride byte offset), descriptor version 1
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(2048 >> 4) << 32) | (1ull << 46);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
// bounded wait for the phase of the given parity to complete; false when the CTA is giving up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < TC_WAIT_LIMIT; it++) {
        uint32_t ok;
        // try_wait suspends the thread in hardware for a while before it reports "not yet"
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

__device__ __forceinline__ void tmem_ld16(int (&v)[16], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}

struct TcBars {
    uint64_t full[TC_STAGES], empty[TC_STAGES], tfull[TC_TSTAGES], tempty[TC_TSTAGES];
    uint32_t tmem_base;
    int abort_flag;
};

}  // namespace

// MODE 1: 8x8 gemm chain, MODE 2: tiled chain (see the file comment)
template <int MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_q4_K_tcgen05_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ TcBars bars;
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tile0 = (int64_t)blockIdx.y * (TC_ROWS / TILE_ROWS);   // first 32-row weight tile of this CTA
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = (int64_t)blockIdx.x * TC_COLS;
    const int64_t K = acts.k;
    volatile int *abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_STAGES; i++) {
            mbar_init(smem_u32(&bars.full[i]), TC_PROD_WARPS);
            mbar_init(smem_u32(&bars.empty[i]), 1 + TC_EPI_WARPS);
        }
        for (int i = 0; i < TC_TSTAGES; i++) {
            mbar_init(smem_u32(&bars.tfull[i]), 1);
            mbar_init(smem_u32(&bars.tempty[i]), TC_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_EPI_WARPS + TC_PROD_WARPS) {
        // all 512 columns: the CTA's shared memory already keeps a second CTA off this SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;
    pdl_wait();

    if (warp < TC_EPI_WARPS) {
        // ---- epilogue: the f32 chains of weight row 32 q + lane over 16 activation rows ----
        const int q = warp & 3, h = warp >> 2;
        const int64_t tile = tile0 + q;
        const bool row_ok = tile < tiles_n;
        const bool any_col = col0 + 16 * h < m;
        const uint8_t *hdr = tiles + (row_ok ? tile : 0) * (int64_t)nb * 4608 + lane * 16;
        float sumf[16], summin[16];
#pragma unroll
        for (int c = 0; c < 16; c++) sumf[c] = summin[c] = 0.0f;
        for (int b = 0; b < nb; b++) {
            const int s = b % TC_STAGES, t = b % TC_TSTAGES;
            const uint32_t sph = (uint32_t)(b / TC_STAGES) & 1u, tph = (uint32_t)(b / TC_TSTAGES) & 1u;
            uint4 hd = make_uint4(0, 0, 0, 0);
            if (row_ok) hd = *(const uint4 *)(hdr + (int64_t)b * 4608);
            // the whole warp goes on or gives up together: tcgen05.ld below wants it converged
            const bool ready = mbar_wait(smem_u32(&bars.full[s]), sph, abort_flag) && mbar_wait(smem_u32(&bars.tfull[t]), tph, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint8_t *stage = smem + s * TC_STAGE_BYTES;
            const int2 *bp = (const int2 *)(stage + TC_A_BYTES + TC_B_BYTES);             // [pair][column]
            const float *da = (const float *)(stage + TC_A_BYTES + TC_B_BYTES + TC_BP_BYTES);
            // 6-bit scales and mins, one per byte (crates/ggml/src/quants.rs:421-429)
            uint32_t sc[2], mn[2];
            sc[0] = hd.y & 0x3f3f3f3fu;
            mn[0] = hd.z & 0x3f3f3f3fu;
            sc[1] = (hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4);
            mn[1] = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
            const float dw = f16_bits_to_f32((uint16_t)(hd.x & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(hd.x >> 16));
            int s1[16], s2[16];
            if (MODE == 2) {
#pragma unroll
                for (int c = 0; c < 16; c++) s1[c] = s2[c] = 0;
            }
            const uint32_t trow = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(t * 8 * TC_COLS + 16 * h);
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int d0[16], d1[16];
                tmem_ld16(d0, trow + (uint32_t)((2 * g) * TC_COLS));
                tmem_ld16(d1, trow + (uint32_t)((2 * g + 1) * TC_COLS));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (g == 3) {
                    // the accumulator stage is free again once every epilogue warp has read it
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars.tempty[t]));
                }
                if (any_col) {
                    const int sh = 16 * (g & 1);
                    const int s_lo = (sc[g >> 1] >> sh) & 0xff, s_hi = (sc[g >> 1] >> (sh + 8)) & 0xff;
                    const int m_lo = (mn[g >> 1] >> sh) & 0xff, m_hi = (mn[g >> 1] >> (sh + 8)) & 0xff;
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        const int2 bs = bp[g * TC_COLS + 16 * h + c];
                        const int ig = d0[c] * s_lo + d1[c] * s_hi;
                        const int mg = m_lo * bs.x + m_hi * bs.y;
                        if (MODE == 1) {
                            const float dx = da[16 * h + c];
                            sumf[c] = __fmaf_rn((float)ig, __fmul_rn(dw, dx), sumf[c]);
                            summin[c] = __fmaf_rn((float)mg, __fmul_rn(dmw, dx), summin[c]);
                        } else {
                            s1[c] += ig;
                            s2[c] += mg;
                        }
                    }
                }
            }
            if (MODE == 2 && any_col) {
#pragma unroll
                for (int c = 0; c < 16; c++) {
                    float rr = __fmul_rn(dw, (float)s1[c]);
                    rr = __fmaf_rn(-dmw, (float)s2[c], rr);
                    sumf[c] = __fmaf_rn(rr, da[16 * h + c], sumf[c]);
                }
            }
            // this warp is done with the stage's column scales
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.empty[s]));
        }
        const int64_t row = tile * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 16; c++) {
                const int64_t col = col0 + 16 * h + c;
                if (col < m) dst[col * lddst + row] = MODE == 1 ? __fsub_rn(sumf[c], summin[c]) : sumf[c];
            }
        }
    } else if (warp < TC_EPI_WARPS + TC_PROD_WARPS) {
        // ---- producers ----
        const int pw = warp - TC_EPI_WARPS, p = pw * 32 + lane;
        const int64_t tile = tile0 + pw;
        const bool tile_ok = tile < tiles_n;
        const uint8_t *wsrc = tiles + (tile_ok ? tile : 0) * (int64_t)nb * 4608 + 512 + lane * 16;
        const int prow = pw * 32 + lane;
        const uint32_t a_off = (uint32_t)((prow >> 3) * 2048 + (prow & 7) * 16);
        // activation blocks: four 16-byte pieces per thread; consecutive lanes take consecutive columns so that the
        // eight lanes of a store phase fill one 128-byte core matrix
        int64_t bcol[4];
        uint32_t b_off[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = p + 128 * j, col = i & 31, kc = i >> 5;
            const int64_t c = col0 + col;
            bcol[j] = (c < m ? c : m - 1) * K + kc * 16;
            b_off[j] = (uint32_t)((col >> 3) * 2048 + kc * 128 + (col & 7) * 16);
        }
        const int64_t scol = col0 + (p >> 2) < m ? col0 + (p >> 2) : m - 1;   // bsums: column p / 4, pair p % 4
        const int64_t dcol = col0 + lane < m ? col0 + lane : m - 1;
        // the loads of a super-block are issued one step before it is converted
        uint4 w_n[8], y_n[4];
#pragma unroll
        for (int c = 0; c < 8; c++) w_n[c] = tile_ok ? ld_stream16(wsrc + c * 512) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; j++) y_n[j] = *(const uint4 *)(acts.qs + bcol[j]);
        short4 bs_n = *(const short4 *)(acts.bsums + scol * (K / 16) + 4 * (p & 3));
        float dx_n = pw == 0 ? acts.d[dcol * nb] : 0.0f;
        for (int b = 0; b < nb; b++) {
            const int s = b % TC_STAGES;
            const uint32_t sph = (uint32_t)(b / TC_STAGES) & 1u;
            uint4 w[8], y[4];
#pragma unroll
            for (int c = 0; c < 8; c++) w[c] = w_n[c];
#pragma unroll
            for (int j = 0; j < 4; j++) y[j] = y_n[j];
            const short4 bs = bs_n;
            const float dx = dx_n;
            if (b + 1 < nb) {
#pragma unroll
                for (int c = 0; c < 8; c++) w_n[c] = tile_ok ? ld_stream16(wsrc + (int64_t)(b + 1) * 4608 + c * 512) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < 4; j++) y_n[j] = *(const uint4 *)(acts.qs + bcol[j] + (int64_t)(b + 1) * 256);
                bs_n = *(const short4 *)(acts.bsums + scol * (K / 16) + (int64_t)(b + 1) * 16 + 4 * (p & 3));
                if (pw == 0) dx_n = acts.d[dcol * nb + b + 1];
            }
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.empty[s]), sph ^ 1u, abort_flag))) break;
            uint8_t *stage = smem + s * TC_STAGE_BYTES;
            uint8_t *A = stage + a_off, *B = stage + TC_A_BYTES;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                // 16-byte piece c of the row: low nibbles = K chunk (c & 1) of sub-block 2 (c / 2), high nibbles of 2 (c / 2) + 1
                const int kc_lo = 4 * (c >> 1) + (c & 1), kc_hi = kc_lo + 2;
                uint4 lo, hi;
                lo.x = w[c].x & 0x0f0f0f0fu; lo.y = w[c].y & 0x0f0f0f0fu; lo.z = w[c].z & 0x0f0f0f0fu; lo.w = w[c].w & 0x0f0f0f0fu;
                hi.x = (w[c].x >> 4) & 0x0f0f0f0fu; hi.y = (w[c].y >> 4) & 0x0f0f0f0fu;
                hi.z = (w[c].z >> 4) & 0x0f0f0f0fu; hi.w = (w[c].w >> 4) & 0x0f0f0f0fu;
                *(uint4 *)(A + kc_lo * 128) = lo;
                *(uint4 *)(A + kc_hi * 128) = hi;
            }
#pragma unroll
            for (int j = 0; j < 4; j++) *(uint4 *)(B + b_off[j]) = y[j];
            int2 *bp = (int2 *)(stage + TC_A_BYTES + TC_B_BYTES);
            bp[(p & 3) * TC_COLS + (p >> 2)] = make_int2((int)bs.x + (int)bs.y, (int)bs.z + (int)bs.w);
            if (pw == 0) ((float *)(stage + TC_A_BYTES + TC_B_BYTES + TC_BP_BYTES))[lane] = dx;
            // make the stores visible to the tensor core's (async proxy) reads, then hand the stage over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.full[s]));
        }
    } else if (lane == 0) {
        // ---- MMA issue ----
        for (int b = 0; b < nb; b++) {
            const int s = b % TC_STAGES, t = b % TC_TSTAGES;
            const uint32_t sph = (uint32_t)(b / TC_STAGES) & 1u, tph = (uint32_t)(b / TC_TSTAGES) & 1u;
            if (!mbar_wait(smem_u32(&bars.full[s]), sph, abort_flag)) break;
            if (!mbar_wait(smem_u32(&bars.tempty[t]), tph ^ 1u, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = smem_u32(smem + s * TC_STAGE_BYTES), b_base = a_base + TC_A_BYTES;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint64_t adesc = smem_desc(a_base + j * 256), bdesc = smem_desc(b_base + j * 256);
                const uint32_t d_tmem = tmem + (uint32_t)(t * 8 * TC_COLS + j * TC_COLS);
                asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
                             "l"(adesc), "l"(bdesc), "r"(TC_IDESC), "r"(0)
                             : "memory");
            }
            // both arrive when the eight MMAs above have completed: operands consumed, accumulators ready
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.empty[s])) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.tfull[t])) : "memory");
        }
    }
    // ---- teardown: every role has left its loop (finished, or gave up) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_EPI_WARPS + TC_PROD_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, TC_ERR_WAIT);
}

// ---- the 8x8 gemm chain with the sub-block scales folded into the operands ----------------------------
// The integer work of the chain above (two scale multiplies, two min multiplies and two int -> float
// conversions per output element and sub-block pair) is what bounds the kernel, not the tensor pipe.  The
// gemm route only ever needs, per pair g, the two integers
//     ig = s_lo dot_lo + s_hi dot_hi      |ig| <= 2 * 32 * 15 * 127 * 63 < 2^23
//     mg = m_lo bsum_lo + m_hi bsum_hi    |mg| <= 2 * 63 * 32 * 127      < 2^19
// as f32.  Every term and every partial sum is an integer below 2^24, so an f16 x f16 -> f32 MMA whose
// operands are the small integers  s * w  (at most 63 * 15 = 945 < 2048, exact in f16), the activation
// bytes, the mins and the activation 16-element sums (at most 16 * 127 = 2032 < 2048) returns exactly
// f32(ig) and f32(mg), in whatever order the tensor core adds: the producers fold the scales in once
// per weight (one half2 fma per two weights, shared by all 32 activation rows) and the epilogue is left
// with the two fmas of the chain.  The tiled chain sums a whole super-block (up to 2^25) before the
// conversion, so it stays on the integer kernel above.
//   A   [128 rows][256 f16]  s * w, K order within a pair: 16-byte piece p, (low | high) nibbles, bytes (0,2,1,3 ..)
//   B   [32 columns][256 f16] activation bytes in the same order
//   Am  [128 rows][16 f16]   slots 4g, 4g+1 = m_lo of pair g, 4g+2, 4g+3 = m_hi
//   Bm  [4 pairs][32 columns][16 f16]  slots 4g .. 4g+3 = the pair's four 16-element activation sums, rest 0
// per pair: four K = 16 MMAs accumulate ig into 32 tensor-memory columns, one K = 16 MMA writes mg.
namespace {

constexpr int TF_STAGES = 2;
constexpr int TF_A_BYTES = TC_ROWS * 512;
constexpr int TF_B_BYTES = TC_COLS * 512;
constexpr int TF_AM_BYTES = TC_ROWS * 32;
constexpr int TF_BM_BYTES = 4 * TC_COLS * 32;
constexpr int TF_STAGE_BYTES = TF_A_BYTES + TF_B_BYTES + TF_AM_BYTES + TF_BM_BYTES;
constexpr int TF_SMEM_BYTES = TF_STAGES * TF_STAGE_BYTES + 1024;
// kind::f16 instruction descriptor: f32 accumulator, f16 x f16, both operands K-major, N = 32, M = 128
constexpr uint32_t TF_IDESC = (1u << 4) | ((uint32_t)(TC_COLS >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);

__device__ __forceinline__ uint64_t smem_desc_ls(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
// nibbles at bit `shift` of bytes 0 and 2 of the word, times the scale: (1024 + w) s - 1024 s, exact
__device__ __forceinline__ uint32_t scaled_nibbles(uint32_t word, int shift, __half2 s2, __half2 c2) {
    return h2_bits(__hfma2(bits_h2(((word >> shift) & 0x000f000fu) | 0x64006400u), s2, c2));
}
// signed bytes 0 and 2 of the word (after the sign flip u = y ^ 0x80): (1024 + u) - 1152, exact
__device__ __forceinline__ uint32_t signed_bytes(uint32_t u, int shift) {
    return h2_bits(__hsub2(bits_h2(((u >> shift) & 0x00ff00ffu) | 0x64006400u), __float2half2_rn(1152.0f)));
}
__device__ __forceinline__ void tmem_ld16f(float (&v)[16], uint32_t taddr) {
    int r[16];
    tmem_ld16(r, taddr);
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __int_as_float(r[i]);
}

constexpr int TF_WORK_WARPS = 16;                               // every one of them converts and drains
constexpr int TF_THREADS = (TF_WORK_WARPS + 1) * 32;            // + the MMA-issuing warp
constexpr int TF_DA_SLOTS = 4;                                  // ring of activation-scale rows (see the kernel)

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tmem_ld8f(float (&v)[8], uint32_t taddr) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __uint_as_float(r[i]);
}

#define sts128(addr, x_, y_, z_, w_) sts128(addr, x_, y_, z_, w_)

struct TfBars {
    uint64_t full[TF_STAGES], empty[TF_STAGES], tfull[TC_TSTAGES], tempty[TC_TSTAGES];
    float da[TF_DA_SLOTS][TC_COLS];
    uint32_t tmem_base;
    int abort_flag;
};

}  // namespace

// Roles.  The integer kernel above gives every pipeline role its own warps; measured per role, those warps
// spend most of their issue slots polling barriers for one another.  Here all 16 worker warps do the same
// thing in the same order, so they reach each hand-off together: in iteration b every worker converts its
// share of super-block b into the free shared-memory stage (2 weight pieces and 1 activation piece per
// thread, loaded from global memory one iteration ahead), hands the stage to the MMA warp, and then drains
// the accumulators of super-block b - 1 (tensor-memory lanes 32 (w % 4) .. + 31, activation rows
// 8 (w / 4) .. + 7), whose MMAs ran while this iteration's conversion was going on.  Warp 16 only issues
// MMAs and commits.
__global__ void __launch_bounds__(TF_THREADS, 1)
gemm_q4_K_tcgen05_f16_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ TfBars bars;
    pdl_trigger();
    const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int64_t tile0 = (int64_t)blockIdx.y * (TC_ROWS / TILE_ROWS);
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    const int64_t col0 = (int64_t)blockIdx.x * TC_COLS;
    const int64_t K = acts.k;
    volatile int *abort_flag = &bars.abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TF_STAGES; i++) {
            mbar_init(smem_u32(&bars.full[i]), TF_WORK_WARPS);
            mbar_init(smem_u32(&bars.empty[i]), 1);
        }
        for (int i = 0; i < TC_TSTAGES; i++) {
            mbar_init(smem_u32(&bars.tfull[i]), 1);
            mbar_init(smem_u32(&bars.tempty[i]), TF_WORK_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TF_WORK_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;
    pdl_wait();

    if (warp < TF_WORK_WARPS) {
        // ---- conversion share: weight pieces c0 and c0 + 4 of row (tt, lane); activation piece tid; sums for tid < 128 ----
        const int tt = warp & 3, c0 = warp >> 2;
        const bool tile_ok = tile0 + tt < tiles_n;
        const uint8_t *wsrc = tiles + (tile_ok ? tile0 + tt : 0) * (int64_t)nb * 4608 + lane * 16;
        const int prow = tt * 32 + lane;
        const uint32_t a_off = (uint32_t)((prow >> 3) * 4096 + (prow & 7) * 16);
        const uint32_t am_off = (uint32_t)(TF_A_BYTES + TF_B_BYTES + (prow >> 3) * 256 + (prow & 7) * 16);
        // activation piece: column = lane, 16-byte piece kc = warp, so that the eight lanes of a store phase fill one
        // 128-byte core matrix (consecutive columns) instead of hitting the same banks eight times
        const int bcol_i = lane, kc = warp;
        const int64_t bsrc = (col0 + bcol_i < m ? col0 + bcol_i : m - 1) * K + kc * 16;
        // piece kc of the super-block: pair kc / 4, then (low p0, low p1, high p0, high p1) -> chunks 8 g + 4 p + 2 hi
        const uint32_t b_off = (uint32_t)(TF_A_BYTES + (bcol_i >> 3) * 4096 + (bcol_i & 7) * 16 + (8 * (kc >> 2) + 4 * (kc & 1) + 2 * ((kc >> 1) & 1)) * 128);
        const bool has_sum = tid < 128, has_da = tid >= 128 && tid < 128 + TC_COLS;
        const int sg = (tid >> 5) & 3, scol_i = tid & 31;          // sums: pair = warp, column = lane (same reason)
        const int64_t ssrc = (col0 + scol_i < m ? col0 + scol_i : m - 1) * (K / 16) + 4 * sg;
        const uint32_t bm_off = (uint32_t)(TF_A_BYTES + TF_B_BYTES + TF_AM_BYTES + sg * 1024 + (scol_i >> 3) * 256 + (scol_i & 7) * 16);
        const int64_t dsrc = (col0 + (tid & 31) < m ? col0 + (tid & 31) : m - 1) * nb;
        // ---- epilogue share: weight row 32 q + lane, activation rows 8 h .. + 7 ----
        const int q = warp & 3, h = warp >> 2;
        const bool row_ok = tile0 + q < tiles_n;
        const bool any_col = col0 + 8 * h < m;
        const uint8_t *hdr = tiles + (row_ok ? tile0 + q : 0) * (int64_t)nb * 4608 + lane * 16;
        float sumf[8], summin[8];
#pragma unroll
        for (int c = 0; c < 8; c++) sumf[c] = summin[c] = 0.0f;

        // loads of super-block 0
        uint4 hd_n = make_uint4(0, 0, 0, 0), w_n[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, y_n;
        short4 bs_n = make_short4(0, 0, 0, 0);
        float dx_n = 0.0f;
        uint32_t dd_n = 0, dd = 0;
        if (tile_ok) {
            hd_n = *(const uint4 *)(wsrc);
            w_n[0] = ld_stream16(wsrc + 512 + c0 * 512);
            w_n[1] = ld_stream16(wsrc + 512 + (c0 + 4) * 512);
        }
        y_n = *(const uint4 *)(acts.qs + bsrc);
        if (has_sum) bs_n = *(const short4 *)(acts.bsums + ssrc);
        if (has_da) dx_n = acts.d[dsrc];
        if (row_ok) dd_n = *(const uint32_t *)(hdr);

        for (int b = 0; b <= nb; b++) {
            const uint32_t de = dd;   // the epilogue row's (d, dmin) of super-block b - 1
            if (b < nb) {
                const int s = b % TF_STAGES;
                const uint32_t sph = (uint32_t)(b / TF_STAGES) & 1u;
                const uint4 hd = hd_n, w0 = w_n[0], w1 = w_n[1], y = y_n;
                const short4 bs = bs_n;
                const float dx = dx_n;
                dd = dd_n;
                if (b + 1 < nb) {
                    if (tile_ok) {
                        hd_n = *(const uint4 *)(wsrc + (int64_t)(b + 1) * 4608);
                        w_n[0] = ld_stream16(wsrc + (int64_t)(b + 1) * 4608 + 512 + c0 * 512);
                        w_n[1] = ld_stream16(wsrc + (int64_t)(b + 1) * 4608 + 512 + (c0 + 4) * 512);
                    }
                    y_n = *(const uint4 *)(acts.qs + bsrc + (int64_t)(b + 1) * 256);
                    if (has_sum) bs_n = *(const short4 *)(acts.bsums + ssrc + (int64_t)(b + 1) * 16);
                    if (has_da) dx_n = acts.d[dsrc + b + 1];
                    if (row_ok) dd_n = *(const uint32_t *)(hdr + (int64_t)(b + 1) * 4608);
                }
                if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.empty[s]), sph ^ 1u, abort_flag))) break;
                const uint32_t stage = smem + (uint32_t)(s * TF_STAGE_BYTES);
                const uint32_t sc_lo = hd.y & 0x3f3f3f3fu, sc_hi = (hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4);
                if (c0 == 0)
                {
                    const uint32_t mn0 = hd.z & 0x3f3f3f3fu, mn1 = ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4);
                    uint32_t mins[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) mins[j] = h2_bits(__half2half2(__int2half_rn((int)(((j < 4 ? mn0 : mn1) >> (8 * (j & 3))) & 0xff))));
                    sts128(stage + am_off, mins[0], mins[1], mins[2], mins[3]);
                    sts128(stage + am_off + 128, mins[4], mins[5], mins[6], mins[7]);
                }
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    // piece c = c0 + 4 j: pair g = c / 2 (sub-blocks 2 g, 2 g + 1), 16-byte piece pp = c % 2 within it
                    const int c = c0 + 4 * j, g = c >> 1, pp = c & 1;
                    const uint4 w = j ? w1 : w0;
                    const uint32_t scw = j ? sc_hi : sc_lo;                  // sub-blocks 0..3 | 4..7
                    const int s_lo = (scw >> (16 * (g & 1))) & 0xff, s_hi = (scw >> (16 * (g & 1) + 8)) & 0xff;
                    const __half2 sl = __half2half2(__int2half_rn(s_lo)), sh = __half2half2(__int2half_rn(s_hi));
                    const __half2 cl = __half2half2(__int2half_rn(-1024 * s_lo)), ch = __half2half2(__int2half_rn(-1024 * s_hi));
                    const uint32_t dstp = stage + a_off + (uint32_t)((8 * g + 4 * pp) * 128);
                    sts128(dstp, scaled_nibbles(w.x, 0, sl, cl), scaled_nibbles(w.x, 8, sl, cl), scaled_nibbles(w.y, 0, sl, cl),
                           scaled_nibbles(w.y, 8, sl, cl));
                    sts128(dstp + 128, scaled_nibbles(w.z, 0, sl, cl), scaled_nibbles(w.z, 8, sl, cl), scaled_nibbles(w.w, 0, sl, cl),
                           scaled_nibbles(w.w, 8, sl, cl));
                    sts128(dstp + 256, scaled_nibbles(w.x, 4, sh, ch), scaled_nibbles(w.x, 12, sh, ch), scaled_nibbles(w.y, 4, sh, ch),
                           scaled_nibbles(w.y, 12, sh, ch));
                    sts128(dstp + 384, scaled_nibbles(w.z, 4, sh, ch), scaled_nibbles(w.z, 12, sh, ch), scaled_nibbles(w.w, 4, sh, ch),
                           scaled_nibbles(w.w, 12, sh, ch));
                }
                {
                    const uint32_t u0 = y.x ^ 0x80808080u, u1 = y.y ^ 0x80808080u, u2 = y.z ^ 0x80808080u, u3 = y.w ^ 0x80808080u;
                    sts128(stage + b_off, signed_bytes(u0, 0), signed_bytes(u0, 8), signed_bytes(u1, 0), signed_bytes(u1, 8));
                    sts128(stage + b_off + 128, signed_bytes(u2, 0), signed_bytes(u2, 8), signed_bytes(u3, 0), signed_bytes(u3, 8));
                }
                if (has_sum) {
                    const uint32_t xy = h2_bits(__halves2half2(__short2half_rn(bs.x), __short2half_rn(bs.y)));
                    const uint32_t zw = h2_bits(__halves2half2(__short2half_rn(bs.z), __short2half_rn(bs.w)));
                    const bool odd = sg & 1, second = sg >> 1;
                    const uint32_t v0 = odd ? 0u : xy, v1 = odd ? 0u : zw, v2 = odd ? xy : 0u, v3 = odd ? zw : 0u;
                    sts128(stage + bm_off, second ? 0u : v0, second ? 0u : v1, second ? 0u : v2, second ? 0u : v3);
                    sts128(stage + bm_off + 128, second ? v0 : 0u, second ? v1 : 0u, second ? v2 : 0u, second ? v3 : 0u);
                }
                // the activation scales of super-block b, read by every worker in the next iteration; slot b % 4 is
                // rewritten in iteration b + 4, which no worker reaches before all have drained super-block b
                if (has_da) bars.da[b % TF_DA_SLOTS][tid & 31] = dx;
                // make the stores visible to the tensor core's (async proxy) reads, then hand the stage over
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars.full[s]));
            }
            if (b >= 1) {
                // ---- drain super-block e = b - 1: sumf = fma(f32(ig), d d_x, sumf); summin = fma(f32(mg), dmin d_x, summin) ----
                const int e = b - 1, t = e % TC_TSTAGES;
                const uint32_t tph = (uint32_t)(e / TC_TSTAGES) & 1u;
                // full[] of that super-block completed long ago; waiting on it orders this warp's reads of da[] after the store
                const bool ready = mbar_wait(smem_u32(&bars.full[e % TF_STAGES]), (uint32_t)(e / TF_STAGES) & 1u, abort_flag) &&
                                   mbar_wait(smem_u32(&bars.tfull[t]), tph, abort_flag);
                if (!__all_sync(0xffffffffu, ready)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float dw = f16_bits_to_f32((uint16_t)(de & 0xffffu)), dmw = f16_bits_to_f32((uint16_t)(de >> 16));
                float sd[8], sm[8];
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    const float dxe = bars.da[e % TF_DA_SLOTS][8 * h + c];
                    sd[c] = __fmul_rn(dw, dxe);
                    sm[c] = __fmul_rn(dmw, dxe);
                }
                const uint32_t trow = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(t * 8 * TC_COLS + 8 * h);
#pragma unroll
                for (int gp = 0; gp < 2; gp++) {
                    float ig0[8], mg0[8], ig1[8], mg1[8];
                    tmem_ld8f(ig0, trow + (uint32_t)((2 * gp) * TC_COLS));
                    tmem_ld8f(mg0, trow + (uint32_t)((4 + 2 * gp) * TC_COLS));
                    tmem_ld8f(ig1, trow + (uint32_t)((2 * gp + 1) * TC_COLS));
                    tmem_ld8f(mg1, trow + (uint32_t)((4 + 2 * gp + 1) * TC_COLS));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (gp == 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars.tempty[t]));
                    }
                    if (any_col) {
#pragma unroll
                        for (int c = 0; c < 8; c++) {
                            sumf[c] = __fmaf_rn(ig0[c], sd[c], sumf[c]);
                            summin[c] = __fmaf_rn(mg0[c], sm[c], summin[c]);
                        }
#pragma unroll
                        for (int c = 0; c < 8; c++) {
                            sumf[c] = __fmaf_rn(ig1[c], sd[c], sumf[c]);
                            summin[c] = __fmaf_rn(mg1[c], sm[c], summin[c]);
                        }
                    }
                }
            }
        }
        const int64_t row = (tile0 + q) * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const int64_t col = col0 + 8 * h + c;
                if (col < m) dst[col * lddst + row] = __fsub_rn(sumf[c], summin[c]);
            }
        }
    } else if (lane == 0) {
        // ---- MMA issue ----
        for (int b = 0; b < nb; b++) {
            const int s = b % TF_STAGES, t = b % TC_TSTAGES;
            const uint32_t sph = (uint32_t)(b / TF_STAGES) & 1u, tph = (uint32_t)(b / TC_TSTAGES) & 1u;
            if (!mbar_wait(smem_u32(&bars.full[s]), sph, abort_flag)) break;
            if (!mbar_wait(smem_u32(&bars.tempty[t]), tph ^ 1u, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = smem + (uint32_t)(s * TF_STAGE_BYTES), b_base = a_base + TF_A_BYTES;
            const uint32_t am_base = b_base + TF_B_BYTES, bm_base = am_base + TF_AM_BYTES;
#pragma unroll
            for (int g = 0; g < 4; g++) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint64_t adesc = smem_desc_ls(a_base + (8 * g + 2 * i) * 128, 128, 4096);
                    const uint64_t bdesc = smem_desc_ls(b_base + (8 * g + 2 * i) * 128, 128, 4096);
                    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(
                                     tmem + (uint32_t)(t * 8 * TC_COLS + g * TC_COLS)),
                                 "l"(adesc), "l"(bdesc), "r"(TF_IDESC), "r"(i)
                                 : "memory");
                }
                const uint64_t amdesc = smem_desc_ls(am_base, 128, 256), bmdesc = smem_desc_ls(bm_base + g * 1024, 128, 256);
                asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(
                                 tmem + (uint32_t)(t * 8 * TC_COLS + (4 + g) * TC_COLS)),
                             "l"(amdesc), "l"(bmdesc), "r"(TF_IDESC), "r"(0)
                             : "memory");
            }
            // both arrive when the MMAs above have completed: operands consumed, accumulators ready
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.empty[s])) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.tfull[t])) : "memory");
        }
    }
    // ---- teardown: every role has left its loop (finished, or gave up) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TF_WORK_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, TC_ERR_WAIT);
}

// B200_GEMM_TCGEN05_F16=1 sends the gemm chain to the f16-operand kernel.  Measured on 4096 x 4096 x 512 it takes
// 160 us against the integer kernel's 145 us: its epilogue is four times cheaper, but every worker converts,
// hands over and drains in sequence, and the per-step hand-off and load latencies (2 operand stages of 88 KB
// are all that fits) are not hidden.  It stays selectable until its pipeline is deeper.
// B200_GEMM_TCGEN05_F16 picks the kernel of the gemm chain: 0 = the integer kernel of this file, 1 = its 32-column
// f16-operand kernel, 2 = the 64-column one (gemm_tcgen05_f16.cu), 3 = the two-pass one (gemm_tcgen05_img.cu);
// 4 = the two-pass one with 128 activation rows per CTA; unset = by estimated time among 0, 3 and 4 (gemm_chain_pick below).
int gemm_tcgen05_f16_choice() {
    static int v = -2;
    if (v == -2) {
        const char *e = getenv("B200_GEMM_TCGEN05_F16");
        v = (e && e[0] >= '0' && e[0] <= '4') ? e[0] - '0' : -1;
    }
    return v;
}

// One CTA per SM in every kernel.  Measured at K = 4096: a wave of CTAs takes 37 us in the integer kernel (128 x 32
// outputs per CTA) and in the 64-column two-pass kernel (128 x 64), 1.6 times that in the 128-column one
// (128 x 128); expanding the operands costs 8.7 us per 4096 x 4096 weights and 5.2 us per 512 x 4096 activations
// (0.235 and 0.14 of a wave).  Returns 0 = integer kernel, 3 = two-pass with 64 columns, 4 = with 128.
int gemm_chain_pick_for(int64_t n, int64_t m, int sm_count) {
    if (sm_count <= 0) sm_count = 148;
    const int64_t gy = (n + 127) / 128, g32 = (m + 31) / 32, g64 = (m + 63) / 64, g128 = (m + 127) / 128;
    const auto waves = [&](int64_t ctas) { return (double)((ctas + sm_count - 1) / sm_count); };
    const double expand = 0.235 * (double)gy / 32.0 + 0.14 * (double)g64 / 8.0 + 0.05;
    const double t_int = waves(gy * g32), t_64 = waves(gy * g64) + expand, t_128 = 1.6 * waves(gy * g128) + expand;
    if (t_int <= t_64 && t_int <= t_128) return 0;
    return t_128 < t_64 ? 4 : 3;
}
static int gemm_chain_pick(int64_t n, int64_t m) {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    if (sms[dev] == 0 && (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0)) sms[dev] = 148;
    return gemm_chain_pick_for(n, m, sms[dev]);
}

// mode: 1 = Q4_K gemm chain, 2 = Q4_K tiled chain
int launch_gemm_tcgen05(int mode, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                        cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    B200_REQUIRE(mode == 1 || mode == 2, "gemm: unknown mode %d", mode);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    int choice = gemm_tcgen05_f16_choice();
    // fast numerics: one tensor-memory drain per super-block instead of the CPU chain's per-pair fused multiply-adds
    // (within 1e-5 of sum |w x|, both routes), from 2048 weight rows (1024 x 4096 x 512: 38.9 us on the exact kernels, 55.9 on
    // the fast one, whose fixed costs a matrix of sixteen tiles does not repay); B200_GEMM_FAST=0 keeps the exact kernels,
    // =2 lifts the row limit (read per call)
    if (choice < 0 && numerics_mode() == 1 && m >= GEMM_FAST_MIN_COLS && !no_scratch_mode()) {
        const char *e = getenv("B200_GEMM_FAST");
        if (!(e && e[0] == '0') && (n >= 2048 || (e && e[0] == '2'))) return launch_gemm_q4_K_fast(n, k, m, tiles, acts, dst, lddst, s);
    }
    if (mode == 1 && choice < 0) choice = gemm_chain_pick(n, m);
    if (no_scratch_mode() && (choice == 3 || choice == 4)) choice = 0;   // the two-pass kernels need the image block
    if (mode == 1 && choice == 2) return launch_gemm_tcgen05_f16x64(n, k, m, tiles, acts, dst, lddst, s);
    if (mode == 1 && choice == 3) return launch_gemm_tcgen05_img(n, k, m, tiles, acts, dst, lddst, s);
    if (mode == 1 && choice == 4) return launch_gemm_tcgen05_img128(n, k, m, tiles, acts, dst, lddst, s);
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_tcgen05_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TF_SMEM_BYTES));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const int nb = (int)(k / GROUP_K);
    const int64_t gx = (m + TC_COLS - 1) / TC_COLS, gy = (n + TC_ROWS - 1) / TC_ROWS;
    B200_REQUIRE(gx < 0x7fffffffLL && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    const dim3 grid((unsigned)gx, (unsigned)gy), block(TC_THREADS);
    if (mode == 1 && choice == 1)
        return launch_pdl(gemm_q4_K_tcgen05_f16_kernel, grid, dim3(TF_THREADS), (size_t)TF_SMEM_BYTES, s, tiles, acts, dst, lddst, n, nb, m, err);
    if (mode == 1) return launch_pdl(gemm_q4_K_tcgen05_kernel<1>, grid, block, (size_t)TC_SMEM_BYTES, s, tiles, acts, dst, lddst, n, nb, m, err);
    return launch_pdl(gemm_q4_K_tcgen05_kernel<2>, grid, block, (size_t)TC_SMEM_BYTES, s, tiles, acts, dst, lddst, n, nb, m, err);
}

}  // namespace b200
