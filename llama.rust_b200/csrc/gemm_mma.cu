// Prompt-shaped mat-mul (tens to thousands of activation rows) for the K-quants: the integer block
// dots run on the tensor cores, the f32 accumulation chains of the mirrored CPU route run in registers.
//
// The CPU routes never add two sub-blocks' integer dots before scaling them: every 32-element (Q4_K) or
// 16-element (Q6_K) sub-block has its own integer scale, and the products enter an f32 chain in a fixed
// order.  So one tensor-core instruction computes exactly one sub-block's dots for a 16-row x 8-column
// patch (mma.sync m16n8k32 / m16n8k16, s8 x s8 -> s32, accumulator cleared each time: the sums are
// exact), and the thread that receives a dot applies the sub-block scale with integer arithmetic and
// feeds the route's f32 chain:
//   Q4_K, 8x8 gemm  (crates/ggml/src/repack.rs:1692-1768)  per super-block and sub-block pair g:
//         sumf = fma(f32(ig[g]), d*d_x, sumf); summin = fma(f32(mg[g]), dmin*d_x, summin); out = sumf - summin
//   Q4_K, tiled     (crates/ggml/src/tiled.rs:823-838)     r = d*f32(s1); r = fma(-dmin, f32(s2), r); out = fma(r, d_x, out)
//   Q6_K, tiled     (crates/ggml/src/tiled.rs:723-839)     r = d*f32(s1); out = fma(r, d_x, out)
// which makes the result bit-identical to the decode kernels' and to the CPU's.
//
// One warp owns one 32-row weight tile x 16 activation rows and walks K super-block by super-block;
// a CTA is 4 tiles x 2 column groups.  Weights come straight from the tile layout: the four lanes that
// share a row read 32 contiguous bytes of it per load, and since a dot product does not care in which
// order its terms are summed, lane t supplies elements 8t..8t+7 of a sub-block (Q4_K) where the
// instruction's nominal layout says 4t..4t+3 and 16+4t..16+4t+3; the activation fragment uses the same
// assignment.  There is no shared memory and no barrier: the only reuse is the L1/L2 hit of the other
// column group's identical weight loads and of the four row tiles' identical activation loads.
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ void mma_s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void mma_s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ uint2 ldg8(const void *p) { return *(const uint2 *)p; }
__device__ __forceinline__ uint32_t ldg4(const void *p) { return *(const uint32_t *)p; }

constexpr int MMA_WARPS = 8;          // 4 row tiles x 2 column groups
constexpr int MMA_COLS = 16;          // activation rows per warp (two n8 patches)

// MODE 1: 8x8 gemm chain, MODE 2: tiled chain (see the file comment)
template <int MODE>
__global__ void __launch_bounds__(MMA_WARPS * 32, 2)
gemm_q4_K_mma_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g8 = lane >> 2, t = lane & 3;
    const int64_t tile = (int64_t)blockIdx.x * 4 + (warp & 3);
    if (tile * TILE_ROWS >= n) return;
    const int64_t col0 = ((int64_t)blockIdx.y * 2 + (warp >> 2)) * MMA_COLS;
    if (col0 >= m) return;
    // this thread's four columns: patch nt, columns 2t and 2t+1 of it; loads clamp to the last valid column
    int64_t colc[2][2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int64_t c = col0 + 8 * nt + 2 * t + j;
            colc[nt][j] = c < m ? c : m - 1;
        }
    // the activation row this lane loads fragments from: patch nt, column g8 of it
    int64_t colb[2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const int64_t c = col0 + 8 * nt + g8;
        colb[nt] = c < m ? c : m - 1;
    }
    float sumf[2][2][4], summin[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) sumf[mt][nt][e] = summin[mt][nt][e] = 0.0f;

    const uint8_t *base = tiles + tile * (int64_t)nb * 4608;
    const int64_t K = acts.k;
    pdl_wait();
    for (int b = 0; b < nb; b++) {
        const uint8_t *chunk = base + (int64_t)b * 4608;
        // column scales of this super-block
        float da[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int j = 0; j < 2; j++) da[nt][j] = acts.d[colc[nt][j] * nb + b];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            // rows ra = 16 mt + g8 and rb = ra + 8: header words (d|dmin, 12 scale bytes)
            const int ra = 16 * mt + g8, rb = ra + 8;
            const uint4 ha = *(const uint4 *)(chunk + ra * 16), hb = *(const uint4 *)(chunk + rb * 16);
            uint32_t sc[2][2], mn[2][2];   // [row a/b][lo4 / hi4], 6-bit values one per byte (crates/ggml/src/quants.rs:421-429)
            sc[0][0] = ha.y & 0x3f3f3f3fu; mn[0][0] = ha.z & 0x3f3f3f3fu;
            sc[0][1] = (ha.w & 0x0f0f0f0fu) | (((ha.y >> 6) & 0x03030303u) << 4);
            mn[0][1] = ((ha.w >> 4) & 0x0f0f0f0fu) | (((ha.z >> 6) & 0x03030303u) << 4);
            sc[1][0] = hb.y & 0x3f3f3f3fu; mn[1][0] = hb.z & 0x3f3f3f3fu;
            sc[1][1] = (hb.w & 0x0f0f0f0fu) | (((hb.y >> 6) & 0x03030303u) << 4);
            mn[1][1] = ((hb.w >> 4) & 0x0f0f0f0fu) | (((hb.z >> 6) & 0x03030303u) << 4);
            const float dw[2] = {f16_bits_to_f32((uint16_t)(ha.x & 0xffffu)), f16_bits_to_f32((uint16_t)(hb.x & 0xffffu))};
            const float dmw[2] = {f16_bits_to_f32((uint16_t)(ha.x >> 16)), f16_bits_to_f32((uint16_t)(hb.x >> 16))};
            int s1[2][4], s2[2][4];   // MODE 2: whole super-block sums per element [nt][e]
            if (MODE == 2) {
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) s1[nt][e] = s2[nt][e] = 0;
            }
#pragma unroll
            for (int g = 0; g < 4; g++) {
                // weights of sub-blocks 2g (low nibbles) and 2g+1 (high nibbles): bytes 32g + 8t .. + 7 of the row
                const uint8_t *wq = chunk + 512 + (2 * g + (t >> 1)) * 512 + 8 * (t & 1);
                const uint2 wa = ldg8(wq + ra * 16), wb = ldg8(wq + rb * 16);
                int dots[2][2][4];   // [sub][nt][e]
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int8_t *aq = acts.qs + colb[nt] * K + (int64_t)b * 256 + 64 * g + 8 * t;
                    const uint2 y0 = ldg8(aq), y1 = ldg8(aq + 32);
                    mma_s8_k32(dots[0][nt], wa.x & 0x0f0f0f0fu, wb.x & 0x0f0f0f0fu, wa.y & 0x0f0f0f0fu, wb.y & 0x0f0f0f0fu, y0.x, y0.y);
                    mma_s8_k32(dots[1][nt], (wa.x >> 4) & 0x0f0f0f0fu, (wb.x >> 4) & 0x0f0f0f0fu, (wa.y >> 4) & 0x0f0f0f0fu,
                               (wb.y >> 4) & 0x0f0f0f0fu, y1.x, y1.y);
                }
                const int sh = 16 * (g & 1);
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        // bsums of the pair's four 16-element runs -> the two sub-block sums
                        const short4 bs = *(const short4 *)(acts.bsums + colc[nt][j] * (K / 16) + (int64_t)b * 16 + 4 * g);
                        const int bp_lo = (int)bs.x + (int)bs.y, bp_hi = (int)bs.z + (int)bs.w;
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            const int e = 2 * r + j;   // c0,c1: row a; c2,c3: row b
                            const int s_lo = (sc[r][g >> 1] >> sh) & 0xff, s_hi = (sc[r][g >> 1] >> (sh + 8)) & 0xff;
                            const int m_lo = (mn[r][g >> 1] >> sh) & 0xff, m_hi = (mn[r][g >> 1] >> (sh + 8)) & 0xff;
                            const int ig = dots[0][nt][e] * s_lo + dots[1][nt][e] * s_hi;
                            const int mg = m_lo * bp_lo + m_hi * bp_hi;
                            if (MODE == 1) {
                                const float sd = __fmul_rn(dw[r], da[nt][j]), sm = __fmul_rn(dmw[r], da[nt][j]);
                                sumf[mt][nt][e] = __fmaf_rn((float)ig, sd, sumf[mt][nt][e]);
                                summin[mt][nt][e] = __fmaf_rn((float)mg, sm, summin[mt][nt][e]);
                            } else {
                                s1[nt][e] += ig;
                                s2[nt][e] += mg;
                            }
                        }
                    }
                }
            }
            if (MODE == 2) {
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int r = e >> 1, j = e & 1;
                        float rr = __fmul_rn(dw[r], (float)s1[nt][e]);
                        rr = __fmaf_rn(-dmw[r], (float)s2[nt][e], rr);
                        sumf[mt][nt][e] = __fmaf_rn(rr, da[nt][j], sumf[mt][nt][e]);
                    }
            }
        }
    }
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int64_t row = tile * TILE_ROWS + 16 * mt + g8 + 8 * (e >> 1);
                const int64_t col = col0 + 8 * nt + 2 * t + (e & 1);
                if (row < n && col < m)
                    dst[col * lddst + row] = MODE == 1 ? __fsub_rn(sumf[mt][nt][e], summin[mt][nt][e]) : sumf[mt][nt][e];
            }
}

// Q6_K tiled chain.  Chunk layout: ql 8 sub-chunks | qh 4 | scales 1 | d; sub-block (n, q, h) of the
// super-block = elements 128 n + 32 q + 16 h .. + 15 with ql byte 64 n + 32 (q & 1) + 16 h + l (low nibble for
// q < 2, high for q >= 2) and bits 2q, 2q+1 of qh byte 32 n + 16 h + l (crates/ggml/src/quants.rs:585-612).
// The 6-bit values go to the tensor core as q - 32, so a dot is already sum (q - 32) y.
__global__ void __launch_bounds__(MMA_WARPS * 32, 2)
gemm_q6_K_mma_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m) {
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g8 = lane >> 2, t = lane & 3;
    const int64_t tile = (int64_t)blockIdx.x * 4 + (warp & 3);
    if (tile * TILE_ROWS >= n) return;
    const int64_t col0 = ((int64_t)blockIdx.y * 2 + (warp >> 2)) * MMA_COLS;
    if (col0 >= m) return;
    int64_t colc[2][2], colb[2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int64_t c = col0 + 8 * nt + 2 * t + j;
            colc[nt][j] = c < m ? c : m - 1;
        }
        const int64_t c = col0 + 8 * nt + g8;
        colb[nt] = c < m ? c : m - 1;
    }
    float acc[2][2][4];
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[mt][nt][e] = 0.0f;
    const uint8_t *base = tiles + tile * (int64_t)nb * 6720;
    const int64_t K = acts.k;
    pdl_wait();
    for (int b = 0; b < nb; b++) {
        const uint8_t *chunk = base + (int64_t)b * 6720;
        float da[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int j = 0; j < 2; j++) da[nt][j] = acts.d[colc[nt][j] * nb + b];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            const int ra = 16 * mt + g8, rb = ra + 8;
            const uint4 sa = *(const uint4 *)(chunk + 6144 + ra * 16), sb = *(const uint4 *)(chunk + 6144 + rb * 16);   // 16 int8 scales
            const float dw[2] = {f16_bits_to_f32(*(const uint16_t *)(chunk + 6656 + ra * 2)),
                                 f16_bits_to_f32(*(const uint16_t *)(chunk + 6656 + rb * 2))};
            int s1[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) s1[nt][e] = 0;
#pragma unroll
            for (int nh = 0; nh < 4; nh++) {   // (n, h): four sub-blocks q = 0..3 share these three loads per row
                const int nn = nh >> 1, h = nh & 1;
                const uint8_t *pa = chunk + (4 * nn + h) * 512 + 4 * t, *pb = chunk + (4 * nn + 2 + h) * 512 + 4 * t;
                const uint8_t *ph = chunk + 4096 + (2 * nn + h) * 512 + 4 * t;
                const uint32_t Aa = ldg4(pa + ra * 16), Ba = ldg4(pb + ra * 16), Ha = ldg4(ph + ra * 16);
                const uint32_t Ab = ldg4(pa + rb * 16), Bb = ldg4(pb + rb * 16), Hb = ldg4(ph + rb * 16);
                uint32_t wa[4], wb[4];
                wa[0] = (Aa & 0x0f0f0f0fu) | ((Ha << 4) & 0x30303030u);
                wa[1] = (Ba & 0x0f0f0f0fu) | ((Ha << 2) & 0x30303030u);
                wa[2] = ((Aa >> 4) & 0x0f0f0f0fu) | (Ha & 0x30303030u);
                wa[3] = ((Ba >> 4) & 0x0f0f0f0fu) | ((Ha >> 2) & 0x30303030u);
                wb[0] = (Ab & 0x0f0f0f0fu) | ((Hb << 4) & 0x30303030u);
                wb[1] = (Bb & 0x0f0f0f0fu) | ((Hb << 2) & 0x30303030u);
                wb[2] = ((Ab >> 4) & 0x0f0f0f0fu) | (Hb & 0x30303030u);
                wb[3] = ((Bb >> 4) & 0x0f0f0f0fu) | ((Hb >> 2) & 0x30303030u);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t a0 = __vsub4(wa[q], 0x20202020u), a1 = __vsub4(wb[q], 0x20202020u);
                    const int sub = 8 * nn + 2 * q + h;   // scale index = element / 16
                    const int sca = (int)(int8_t)((sub < 4 ? sa.x : sub < 8 ? sa.y : sub < 12 ? sa.z : sa.w) >> (8 * (sub & 3)));
                    const int scb = (int)(int8_t)((sub < 4 ? sb.x : sub < 8 ? sb.y : sub < 12 ? sb.z : sb.w) >> (8 * (sub & 3)));
#pragma unroll
                    for (int nt = 0; nt < 2; nt++) {
                        const uint32_t y = ldg4(acts.qs + colb[nt] * K + (int64_t)b * 256 + 128 * nn + 32 * q + 16 * h + 4 * t);
                        int d[4];
                        mma_s8_k16(d, a0, a1, y);
                        s1[nt][0] += sca * d[0];
                        s1[nt][1] += sca * d[1];
                        s1[nt][2] += scb * d[2];
                        s1[nt][3] += scb * d[3];
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float rr = __fmul_rn(dw[e >> 1], (float)s1[nt][e]);
                    acc[mt][nt][e] = __fmaf_rn(rr, da[nt][e & 1], acc[mt][nt][e]);
                }
        }
    }
#pragma unroll
    for (int mt = 0; mt < 2; mt++)
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int64_t row = tile * TILE_ROWS + 16 * mt + g8 + 8 * (e >> 1);
                const int64_t col = col0 + 8 * nt + 2 * t + (e & 1);
                if (row < n && col < m) dst[col * lddst + row] = acc[mt][nt][e];
            }
}

// ---- a handful of activation rows (batched decode: 8 to 31) ----------------------------------------------
// With 16 columns the kernel above has one warp per 32-row tile walk all of K: 128 warps on the whole GPU for a
// 4096-row matrix.  Here a CTA owns one row tile x 16 columns and its SMALL_WIN (8 or 16) warps split K: in every
// window of SMALL_WIN super-blocks warp w computes super-block w's sub-block dots with mma.sync, scales them
// (integers) and leaves ig[col][row][pair] in shared memory with the rows' headers, the columns' activation sums
// and scales; after a barrier the CTA's threads (one (row, col) each with 16 warps, two with 8) run the 8x8 gemm
// chain over the window in K order, so the result is the one the kernel above and the CPU produce.  A warp's
// window is one round trip to memory followed by its arithmetic, and the warps of a CTA take it in step, so the
// time is windows x (latency + issue): 16 warps halve the windows of a long row (K of 4096 is one window).
struct SmallStage {
    int4 ig[16][33];        // scaled pair dots [column][row] = {pair 0..3}; 33 entries per column: a store's quarter warp (rows g8, g8 + 1 of four column pairs) and a chain load's (eight rows of one column) each cover 32 different banks
    uint4 hdr[32];          // the rows' (d, dmin as f32 bits, mins 0..3, mins 4..7 one per byte)
    uint4 bp[16];           // the columns' sub-block sums, two 16-bit sums per word = one sub-block pair
    float da[16];           // the columns' super-block scales
};
// c + (low half of a) * (byte 0 of b) + (high half of a) * (byte 1 of b), halves signed, bytes unsigned; _hi: bytes 2 and 3
__device__ __forceinline__ int dp2a_lo_su(uint32_t a, uint32_t b) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(0));
    return d;
}
__device__ __forceinline__ int dp2a_hi_su(uint32_t a, uint32_t b) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(0));
    return d;
}
// up to three matrices of one row length against the same activation rows in one launch: matrix e owns the CTAs
// tile_start[e] .. tile_start[e + 1] of the grid's x range
struct SmallMats {
    const uint8_t *tiles[3];
    float *dst[3];
    int64_t n[3], lddst[3];
    int tile_start[4];
};
template <int SMALL_WIN>
__global__ void __launch_bounds__(SMALL_WIN * 32, 16 / SMALL_WIN)
gemm_q4_K_small_kernel(const SmallMats mats, ActView acts, int nb, int64_t m) {
    extern __shared__ __align__(16) unsigned char small_sm[];
    SmallStage *st = (SmallStage *)small_sm;   // [SMALL_WIN]
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g8 = lane >> 2, t = lane & 3;
    const int me = (int)blockIdx.x >= mats.tile_start[2] ? 2 : (int)blockIdx.x >= mats.tile_start[1] ? 1 : 0;
    const uint8_t *tiles = mats.tiles[me];
    float *dst = mats.dst[me];
    const int64_t n = mats.n[me], lddst = mats.lddst[me];
    const int64_t tile = (int)blockIdx.x - mats.tile_start[me];
    const int64_t col0 = (int64_t)blockIdx.y * 16;
    const int64_t K = acts.k;
    // activation rows this lane loads fragments from (patch nt, column g8 of it), clamped to the last valid one
    int64_t colb[2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const int64_t c = col0 + 8 * nt + g8;
        colb[nt] = c < m ? c : m - 1;
    }
    const uint8_t *base = tiles + tile * (int64_t)nb * 4608;
    // chain threads: row cr, columns cc (and cc + 8 with 8 warps)
    constexpr int NJ = 16 / SMALL_WIN;
    const int cr = threadIdx.x & 31, cc = threadIdx.x >> 5;
    float sumf[NJ], summin[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) sumf[j] = summin[j] = 0.0f;
    pdl_wait();
    for (int w0 = 0; w0 < nb; w0 += SMALL_WIN) {
        const int b = w0 + warp;
        if (b < nb) {
            SmallStage &s = st[warp];
            const uint8_t *chunk = base + (int64_t)b * 4608;
            if (b + SMALL_WIN < nb) {   // the warp's super-block of the next window on its way to L2 (36 lines)
                const uint8_t *nx = chunk + SMALL_WIN * 4608;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + lane * 128));
                if (lane < 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + 4096 + lane * 128));
            }
            {   // row `lane`: d, dmin as f32 and the eight 6-bit mins one per byte (crates/ggml/src/quants.rs:421-429), for the chain threads
                const uint4 hd = *(const uint4 *)(chunk + lane * 16);
                s.hdr[lane] = make_uint4(__float_as_uint(f16_bits_to_f32((uint16_t)(hd.x & 0xffffu))), __float_as_uint(f16_bits_to_f32((uint16_t)(hd.x >> 16))),
                                         hd.z & 0x3f3f3f3fu, ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4));
            }
            if (lane < 16) {
                const int64_t c = col0 + lane < m ? col0 + lane : m - 1;
                s.da[lane] = acts.d[c * nb + b];
            }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int i = lane + 32 * j, col = i >> 2, g = i & 3;   // 16 columns x 4 sub-block pairs
                const int64_t c = col0 + col < m ? col0 + col : m - 1;
                const short4 s4 = *(const short4 *)(acts.bsums + c * (K / 16) + (int64_t)b * 16 + 4 * g);
                ((uint32_t *)&s.bp[col])[g] = (uint32_t)((int)s4.x + (int)s4.y) & 0xffffu | (uint32_t)((int)s4.z + (int)s4.w) << 16;
            }
            // every load of the super-block first (weight fragments of both row halves, activation fragments of both
            // column patches): 64 registers of independent loads in flight per lane, then the arithmetic
            uint2 wa[2][4], wb[2][4], ya[4][2][2];
            uint4 hh[2][2];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int ra = 16 * mt + g8, rb = ra + 8;
                hh[mt][0] = *(const uint4 *)(chunk + ra * 16);
                hh[mt][1] = *(const uint4 *)(chunk + rb * 16);
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const uint8_t *wq = chunk + 512 + (2 * g + (t >> 1)) * 512 + 8 * (t & 1);
                    wa[mt][g] = ldg8(wq + ra * 16);
                    wb[mt][g] = ldg8(wq + rb * 16);
                }
            }
#pragma unroll
            for (int g = 0; g < 4; g++)
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int8_t *aq = acts.qs + colb[nt] * K + (int64_t)b * 256 + 64 * g + 8 * t;
                    ya[g][nt][0] = ldg8(aq);
                    ya[g][nt][1] = ldg8(aq + 32);
                }
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int ra = 16 * mt + g8, rb = ra + 8;
                const uint4 ha = hh[mt][0], hb = hh[mt][1];
                uint32_t sc[2][2];   // [row a/b][sub-blocks 0..3 / 4..7], 6-bit scales one per byte (crates/ggml/src/quants.rs:421-429)
                sc[0][0] = ha.y & 0x3f3f3f3fu;
                sc[0][1] = (ha.w & 0x0f0f0f0fu) | (((ha.y >> 6) & 0x03030303u) << 4);
                sc[1][0] = hb.y & 0x3f3f3f3fu;
                sc[1][1] = (hb.w & 0x0f0f0f0fu) | (((hb.y >> 6) & 0x03030303u) << 4);
                int v[2][4][4];   // [column patch][accumulator][pair]
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const uint2 va = wa[mt][g], vb = wb[mt][g];
                    const int sh = 16 * (g & 1);
                    int s_lo[2], s_hi[2];
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        s_lo[r] = (sc[r][g >> 1] >> sh) & 0xff;
                        s_hi[r] = (sc[r][g >> 1] >> (sh + 8)) & 0xff;
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; nt++) {
                        const uint2 y0 = ya[g][nt][0], y1 = ya[g][nt][1];
                        int d0[4], d1[4];
                        mma_s8_k32(d0, va.x & 0x0f0f0f0fu, vb.x & 0x0f0f0f0fu, va.y & 0x0f0f0f0fu, vb.y & 0x0f0f0f0fu, y0.x, y0.y);
                        mma_s8_k32(d1, (va.x >> 4) & 0x0f0f0f0fu, (vb.x >> 4) & 0x0f0f0f0fu, (va.y >> 4) & 0x0f0f0f0fu,
                                   (vb.y >> 4) & 0x0f0f0f0fu, y1.x, y1.y);
#pragma unroll
                        for (int e = 0; e < 4; e++) v[nt][e][g] = d0[e] * s_lo[e >> 1] + d1[e] * s_hi[e >> 1];   // c0, c1: row a; c2, c3: row b
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        s.ig[8 * nt + 2 * t + (e & 1)][(e >> 1) ? rb : ra] = make_int4(v[nt][e][0], v[nt][e][1], v[nt][e][2], v[nt][e][3]);
            }
        }
        __syncthreads();
        const int wn = nb - w0 < SMALL_WIN ? nb - w0 : SMALL_WIN;
        for (int w = 0; w < wn; w++) {
            const SmallStage &s = st[w];
            const uint4 hd = s.hdr[cr];
            const uint32_t mn_lo = hd.z, mn_hi = hd.w;
            const float dw = __uint_as_float(hd.x), dmw = __uint_as_float(hd.y);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int c = cc + SMALL_WIN * j;
                const float da = s.da[c];
                const float sd = __fmul_rn(dw, da), sm = __fmul_rn(dmw, da);
                const int4 ig = s.ig[c][cr];
                const uint4 bp = s.bp[c];
                // pair g: mins 2g and 2g + 1 times the two sub-blocks' activation sums
                const int mg0 = dp2a_lo_su(bp.x, mn_lo), mg1 = dp2a_hi_su(bp.y, mn_lo), mg2 = dp2a_lo_su(bp.z, mn_hi), mg3 = dp2a_hi_su(bp.w, mn_hi);
                sumf[j] = __fmaf_rn((float)ig.x, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.y, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.z, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.w, sd, sumf[j]);
                summin[j] = __fmaf_rn((float)mg0, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg1, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg2, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg3, sm, summin[j]);
            }
        }
        __syncthreads();
    }
    const int64_t row = tile * TILE_ROWS + cr;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int64_t col = col0 + cc + SMALL_WIN * j;
        if (row < n && col < m) {
            const float v = __fsub_rn(sumf[j], summin[j]);
            dst[col * lddst + row] = v;
            if (acts.sum) acts.sum[col * acts.ld_sum + row] = __fadd_rn(v, acts.addend[col * acts.ld_addend + row]);
        }
    }
}

// The Q6_K tiled chain the same way: warp w leaves r = d * f32(s1) of super-block w for its 32 x 16 patch, the
// chain threads add fma(r, d_x, out) in K order.
struct SmallStageQ6 {
    float rr[16][33];       // [column][row]
    float da[16];
};
template <int SMALL_WIN>
__global__ void __launch_bounds__(SMALL_WIN * 32, 16 / SMALL_WIN)
gemm_q6_K_small_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m) {
    __shared__ SmallStageQ6 st[SMALL_WIN];
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g8 = lane >> 2, t = lane & 3;
    const int64_t tile = blockIdx.x;
    const int64_t col0 = (int64_t)blockIdx.y * 16;
    const int64_t K = acts.k;
    int64_t colb[2];
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        const int64_t c = col0 + 8 * nt + g8;
        colb[nt] = c < m ? c : m - 1;
    }
    const uint8_t *base = tiles + tile * (int64_t)nb * 6720;
    constexpr int NJ = 16 / SMALL_WIN;
    const int cr = threadIdx.x & 31, cc = threadIdx.x >> 5;
    float out[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) out[j] = 0.0f;
    pdl_wait();
    for (int w0 = 0; w0 < nb; w0 += SMALL_WIN) {
        const int b = w0 + warp;
        if (b < nb) {
            SmallStageQ6 &s = st[warp];
            const uint8_t *chunk = base + (int64_t)b * 6720;
            if (b + SMALL_WIN < nb) {   // the warp's super-block of the next window on its way to L2 (53 lines)
                const uint8_t *nx = chunk + SMALL_WIN * 6720;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + lane * 128));
                if (lane < 21) asm volatile("prefetch.global.L2 [%0];" ::"l"(nx + 4096 + lane * 128));
            }
            if (lane < 16) {
                const int64_t c = col0 + lane < m ? col0 + lane : m - 1;
                s.da[lane] = acts.d[c * nb + b];
            }
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int ra = 16 * mt + g8, rb = ra + 8;
                const uint4 sa = *(const uint4 *)(chunk + 6144 + ra * 16), sb = *(const uint4 *)(chunk + 6144 + rb * 16);   // 16 int8 scales
                const float dw[2] = {f16_bits_to_f32(*(const uint16_t *)(chunk + 6656 + ra * 2)),
                                     f16_bits_to_f32(*(const uint16_t *)(chunk + 6656 + rb * 2))};
                int s1[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++) s1[nt][e] = 0;
#pragma unroll
                for (int nh = 0; nh < 4; nh++) {
                    const int nn = nh >> 1, h = nh & 1;
                    const uint8_t *pa = chunk + (4 * nn + h) * 512 + 4 * t, *pb = chunk + (4 * nn + 2 + h) * 512 + 4 * t;
                    const uint8_t *ph = chunk + 4096 + (2 * nn + h) * 512 + 4 * t;
                    const uint32_t Aa = ldg4(pa + ra * 16), Ba = ldg4(pb + ra * 16), Ha = ldg4(ph + ra * 16);
                    const uint32_t Ab = ldg4(pa + rb * 16), Bb = ldg4(pb + rb * 16), Hb = ldg4(ph + rb * 16);
                    uint32_t wa[4], wb[4];
                    wa[0] = (Aa & 0x0f0f0f0fu) | ((Ha << 4) & 0x30303030u);
                    wa[1] = (Ba & 0x0f0f0f0fu) | ((Ha << 2) & 0x30303030u);
                    wa[2] = ((Aa >> 4) & 0x0f0f0f0fu) | (Ha & 0x30303030u);
                    wa[3] = ((Ba >> 4) & 0x0f0f0f0fu) | ((Ha >> 2) & 0x30303030u);
                    wb[0] = (Ab & 0x0f0f0f0fu) | ((Hb << 4) & 0x30303030u);
                    wb[1] = (Bb & 0x0f0f0f0fu) | ((Hb << 2) & 0x30303030u);
                    wb[2] = ((Ab >> 4) & 0x0f0f0f0fu) | (Hb & 0x30303030u);
                    wb[3] = ((Bb >> 4) & 0x0f0f0f0fu) | ((Hb >> 2) & 0x30303030u);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t a0 = __vsub4(wa[q], 0x20202020u), a1 = __vsub4(wb[q], 0x20202020u);
                        const int sub = 8 * nn + 2 * q + h;   // scale index = element / 16
                        const int sca = (int)(int8_t)((sub < 4 ? sa.x : sub < 8 ? sa.y : sub < 12 ? sa.z : sa.w) >> (8 * (sub & 3)));
                        const int scb = (int)(int8_t)((sub < 4 ? sb.x : sub < 8 ? sb.y : sub < 12 ? sb.z : sb.w) >> (8 * (sub & 3)));
#pragma unroll
                        for (int nt = 0; nt < 2; nt++) {
                            const uint32_t y = ldg4(acts.qs + colb[nt] * K + (int64_t)b * 256 + 128 * nn + 32 * q + 16 * h + 4 * t);
                            int d[4];
                            mma_s8_k16(d, a0, a1, y);
                            s1[nt][0] += sca * d[0];
                            s1[nt][1] += sca * d[1];
                            s1[nt][2] += scb * d[2];
                            s1[nt][3] += scb * d[3];
                        }
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 2; nt++)
#pragma unroll
                    for (int e = 0; e < 4; e++)
                        s.rr[8 * nt + 2 * t + (e & 1)][(e >> 1) ? rb : ra] = __fmul_rn(dw[e >> 1], (float)s1[nt][e]);
            }
        }
        __syncthreads();
        const int wn = nb - w0 < SMALL_WIN ? nb - w0 : SMALL_WIN;
        for (int w = 0; w < wn; w++) {
            const SmallStageQ6 &s = st[w];
#pragma unroll
            for (int j = 0; j < NJ; j++) out[j] = __fmaf_rn(s.rr[cc + SMALL_WIN * j][cr], s.da[cc + SMALL_WIN * j], out[j]);
        }
        __syncthreads();
    }
    const int64_t row = tile * TILE_ROWS + cr;
#pragma unroll
    for (int j = 0; j < NJ; j++) {
        const int64_t col = col0 + cc + SMALL_WIN * j;
        if (row < n && col < m) {
            dst[col * lddst + row] = out[j];
            if (acts.sum) acts.sum[col * acts.ld_sum + row] = __fadd_rn(out[j], acts.addend[col * acts.ld_addend + row]);
        }
    }
}

// B200_GEMM_SMALL=0 keeps 8 to 31 activation rows on the one-warp-per-tile kernel
static bool gemm_small_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_GEMM_SMALL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// sixteen warps per CTA (one window per 16 super-blocks, one CTA per SM) while the grid is at most one CTA per SM and the
// rows have 16 super-blocks; eight warps and two CTAs per SM beyond that.  B200_GEMM_SMALL_WIN=8|16 forces one form.
static bool small_wide(int nb, int64_t ctas) {
    static int win_env = -1, sms[64] = {0};
    if (win_env < 0) {
        const char *e = getenv("B200_GEMM_SMALL_WIN");
        win_env = (e && e[0] == '8') ? 8 : (e && e[0] == '1') ? 16 : 0;
    }
    if (win_env) return win_env == 16;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    if (!sms[dev] && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
    return nb >= 16 && ctas <= sms[dev];
}

// count Q4_K matrices (8x8 gemm chain) of row length k against the same 8 to 31 activation rows, one launch
int launch_gemm_small_multi(int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                            const int64_t *lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    B200_REQUIRE(count >= 1 && count <= 3 && m >= 1 && m < 32, "gemm: %d matrices x %lld activation rows do not fit the few-rows kernel", count, (long long)m);
    B200_REQUIRE(count == 1 || !acts.sum, "gemm: the fused add goes with a single matrix");
    {   // the persistent form first; -1: not a case for it
        const int rc = launch_gemm_rows_ring(count, n, k, m, tiles, acts, dst, lddst, s);
        if (rc != -1) return rc;
    }
    const int nb = (int)(k / GROUP_K);
    SmallMats mats;
    int64_t total = 0;
    for (int e = 0; e < 3; e++) {
        const int src = e < count ? e : count - 1;
        mats.tiles[e] = tiles[src];
        mats.dst[e] = dst[src];
        mats.n[e] = n[src];
        mats.lddst[e] = lddst[src];
        mats.tile_start[e] = e < count ? (int)total : 0x7fffffff;
        if (e < count) total += (n[e] + TILE_ROWS - 1) / TILE_ROWS;
    }
    mats.tile_start[3] = (int)total;
    if (total == 0) return B200_STATUS_SUCCESS;
    const int64_t sy = (m + 15) / 16;
    B200_REQUIRE(total < 0x7fffffffLL && sy <= 65535, "gemm: %lld row tiles x %lld is too large for one launch", (long long)total, (long long)m);
    static bool attr_done[64] = {false};   // the attribute belongs to the (function, device) pair
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_small_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(SmallStage) * 8)));
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_small_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(SmallStage) * 16)));
        attr_done[dev] = true;
    }
    const dim3 grid((unsigned)total, (unsigned)sy);
    return small_wide(nb, total * sy) ? launch_pdl(gemm_q4_K_small_kernel<16>, grid, dim3(512), sizeof(SmallStage) * 16, s, mats, acts, nb, m)
                                      : launch_pdl(gemm_q4_K_small_kernel<8>, grid, dim3(256), sizeof(SmallStage) * 8, s, mats, acts, nb, m);
}
bool gemm_small_multi_enabled() { return gemm_small_enabled(); }

// mode: 1 = Q4_K gemm chain, 2 = Q4_K tiled chain, 6 = Q6_K tiled chain
int launch_gemm_mma(int mode, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                    cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    const int nb = (int)(k / GROUP_K);
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    if ((mode == 1 || mode == 6) && m < 32 && gemm_small_enabled()) {
        // a few activation rows: K split over the warps of a CTA, sixteen of them when the row has as many super-blocks
        const int64_t sy = (m + 15) / 16;
        B200_REQUIRE(tiles_n < 0x7fffffffLL && sy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
        const dim3 grid((unsigned)tiles_n, (unsigned)sy);
        if (mode == 6)
            return small_wide(nb, tiles_n * sy) ? launch_pdl(gemm_q6_K_small_kernel<16>, grid, dim3(512), 0, s, tiles, acts, dst, lddst, n, nb, m)
                        : launch_pdl(gemm_q6_K_small_kernel<8>, grid, dim3(256), 0, s, tiles, acts, dst, lddst, n, nb, m);
        const int64_t one = n;
        return launch_gemm_small_multi(1, &one, k, m, &tiles, acts, &dst, &lddst, s);
    }
    const int64_t gx = (tiles_n + 3) / 4, gy = (m + 2 * MMA_COLS - 1) / (2 * MMA_COLS);
    B200_REQUIRE(gx < 0x7fffffffLL && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    const dim3 grid((unsigned)gx, (unsigned)gy), block(MMA_WARPS * 32);
    if (mode == 1) return launch_pdl(gemm_q4_K_mma_kernel<1>, grid, block, 0, s, tiles, acts, dst, lddst, n, nb, m);
    if (mode == 2) return launch_pdl(gemm_q4_K_mma_kernel<2>, grid, block, 0, s, tiles, acts, dst, lddst, n, nb, m);
    if (mode == 6) return launch_pdl(gemm_q6_K_mma_kernel, grid, block, 0, s, tiles, acts, dst, lddst, n, nb, m);
    B200_REQUIRE(false, "gemm: unknown mode %d", mode);
}

}  // namespace b200
