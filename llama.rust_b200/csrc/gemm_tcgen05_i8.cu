// Prompt-shaped mat-mul for Q8_0, Q4_0, MXFP4 and Q6_K weights on the fifth-generation tensor cores: tcgen05.mma
// kind::i8 with the block dots accumulated in tensor memory.  Same pipeline as the Q4_K kernel of gemm_tcgen05.cu
// (one CTA = 128 weight rows x 32 activation rows, one 256-element group of K per step, producer warps that unpack
// the weights to int8 K-major core matrices in shared memory, one thread that issues the MMAs and commits, epilogue
// warps that read the dots back with tcgen05.ld and run the route's f32 chain); what differs per type is the
// unpacking and the chain:
//
//   Q4_0 / MXFP4  8x8 gemm route (crates/ggml/src/repack.rs:3380-3421, :1136-1184): per 32-element block
//                 acc = fma(f32(dot), d_w * d_x, acc).  One MMA (K = 32, accumulator cleared) per block into its
//                 own 32 tensor-memory columns; A holds (nibble - 8), respectively the E2M1 code's value x 2
//                 (crates/ggml/src/quants.rs:660): exact int8.  Bit-identical to the CPU route.
//   Q8_0          the same chain over the whole 32-element dot.  The reference's route (tinyBLAS / row dot,
//                 crates/ggml/src/tinyblas.rs:64-74, vec_dot.rs:732-752) keeps eight lane sums of four elements per
//                 block and adds them at the end, so this kernel differs from it by the f32 summation order
//                 (about 1e-7 of sum |w x|): it serves the library's FAST numerics mode; in EXACT mode Q8_0 prompt
//                 batches stay on the decode kernels' column passes, which reproduce the lanes.
//   Q6_K          tiled route (crates/ggml/src/tiled.rs:723-839): per super-block s1 = sum over 16-element sub-blocks
//                 of scale * (sum q y - 32 bsum), an exact int32, then r = d_w * f32(s1); out = fma(r, d_x, out).
//                 s1 = sum_k w'_k y_k with w'_k = scale_sub(k) * (q_k - 32), |w'| <= 4096: the producers split
//                 w' = 64 hi + lo into two int8 planes (lo in [0, 63], hi in [-64, 64]); eight MMAs accumulate the
//                 hi plane over the super-block into 32 tensor-memory columns, eight the lo plane into 32 more, and
//                 the epilogue forms s1 = 64 hi + lo: two accumulator reads per super-block.  Bit-identical.
//
// Every wait is bounded (mbarrier polls with a limit; on expiry the CTA raises its abort flag, records code 4 in the
// device error word, frees its tensor memory and returns).  No cluster, no multicast.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int TI_ROWS = 128;                 // weight rows per CTA (MMA M)
constexpr int TI_COLS = 32;                  // activation rows per CTA (MMA N)
constexpr int TI_EPI_WARPS = 8, TI_PROD_WARPS = 4;
constexpr int TI_THREADS = (TI_EPI_WARPS + TI_PROD_WARPS + 1) * 32;
constexpr int TI_TSTAGES = 2;                // tensor-memory accumulator stages of 256 columns
constexpr int TI_PLANE_BYTES = TI_ROWS * 256;
constexpr int TI_B_BYTES = TI_COLS * 256;
constexpr int TI_SC_BYTES = 8 * TI_COLS * 4; // activation scales: [block][column] (32-element types) or [column] (Q6_K)
constexpr uint32_t TI_WAIT_LIMIT = 1u << 22;
constexpr int TI_ERR_WAIT = 4;

// kind::i8 instruction descriptor: s32 accumulator, s8 x s8, both operands K-major, N = 32, M = 128
constexpr uint32_t TI_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TI_COLS >> 3) << 17) | ((uint32_t)(TI_ROWS >> 4) << 24);

template <int TYPE>
struct TiTraits;
template <>
struct TiTraits<B200_TYPE_Q8_0> { static constexpr int PLANES = 1, STAGES = 3, CHUNK = 8704; };
template <>
struct TiTraits<B200_TYPE_Q4_0> { static constexpr int PLANES = 1, STAGES = 3, CHUNK = 4608; };
template <>
struct TiTraits<B200_TYPE_MXFP4> { static constexpr int PLANES = 1, STAGES = 3, CHUNK = 4352; };
template <>
struct TiTraits<B200_TYPE_Q6_K> { static constexpr int PLANES = 2, STAGES = 2, CHUNK = 6720; };

template <int TYPE>
struct TiSizes {
    static constexpr int STAGE_BYTES = TiTraits<TYPE>::PLANES * TI_PLANE_BYTES + TI_B_BYTES + TI_SC_BYTES;
    static constexpr int SMEM_BYTES = TiTraits<TYPE>::STAGES * STAGE_BYTES + 1024;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
// shared-memory matrix descriptor, no swizzle: 128 bytes between K-adjacent core matrices, 2048 between 8-row groups
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(2048 >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    for (uint32_t it = 0; it < TI_WAIT_LIMIT; it++) {
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
__device__ __forceinline__ void tmem_ld16(int (&v)[16], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}

// four 4-bit codes (one per byte of x) -> four signed bytes of 2 * E2M1: crates/ggml/src/quants.rs:660
__device__ __forceinline__ uint32_t mxfp4_lut4(uint32_t x) {
    const uint32_t lo = x & 0x07070707u;
    const uint32_t t = lo | (lo >> 4);
    const uint32_t sel = (t & 0xffu) | ((t >> 8) & 0xff00u);
    const uint32_t pos = __byte_perm(0x03020100u, 0x0c080604u, sel);
    const uint32_t neg = __byte_perm(0xfdfeff00u, 0xf4f8fafcu, sel);
    const uint32_t m = ((x & 0x08080808u) >> 3) * 0xffu;
    return (pos & ~m) | (neg & m);
}
// four nibbles (one per byte) minus 8, as signed bytes: no borrow between bytes ((n | 0x80) - 8 keeps bit 7 set, then flip it)
__device__ __forceinline__ uint32_t nibbles_minus8(uint32_t x) { return ((x | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// MUL_MAT_ID, grouped by expert: CTA column blockIdx.x is work item w = up to 32 (token, slot) pairs routed to one
// expert.  work_expert[w] names the expert (-1: an unused item, the CTA leaves at once), col_act[32 w + c] the
// quantized activation row of column c and col_out[32 w + c] the output row (pair index), -1 for the unused columns
// of a short item.  Null work_expert: a plain mat-mul.
struct GroupMap {
    const int *work_expert;
    const int *col_act;
    const int *col_out;
    int64_t expert_bytes;
};

struct TiBars {
    uint64_t full[3], empty[3], tfull[TI_TSTAGES], tempty[TI_TSTAGES];
    uint32_t tmem_base;
    int abort_flag;
};

// Q6_K: the 16 six-bit values v of one 16-byte run times the run's scale, w' = sc (v - 32) in [-4064, 4096], as the
// two int8 planes of w' = 64 hi + lo with lo in [0, 63] and hi in [-64, 64]: with w'' = w' + 4096 (non-negative),
// lo = w'' & 63 and hi = (w'' >> 6) - 64, the subtraction done as + 192 modulo 256 so that no borrow leaves the
// byte.  Two values ride in the 16-bit halves of a word through one multiply: |sc| v <= 128 * 63 and every
// intermediate stay below 2^16, so nothing carries from one half into the other.
__device__ __forceinline__ void q6_planes(const uint4 &v, int sc, uint4 *hi, uint4 *lo) {
    const uint32_t a = (uint32_t)(sc < 0 ? -sc : sc);
    // w'' = 4096 + sc v - 32 sc: base = 4096 - 32 sc (in [32, 8192]), then + |sc| v or - |sc| v
    const uint32_t base = (uint32_t)(4096 - 32 * sc) * 0x00010001u;
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t p02 = (w[i] & 0x003f003fu) * a, p13 = ((w[i] >> 8) & 0x003f003fu) * a;
        const uint32_t w02 = sc < 0 ? base - p02 : base + p02, w13 = sc < 0 ? base - p13 : base + p13;
        l[i] = (w02 & 0x003f003fu) | ((w13 & 0x003f003fu) << 8);
        h[i] = (((w02 >> 6) + 0x00c000c0u) & 0x00ff00ffu) | ((((w13 >> 6) + 0x00c000c0u) & 0x00ff00ffu) << 8);
    }
    *hi = make_uint4(h[0], h[1], h[2], h[3]);
    *lo = make_uint4(l[0], l[1], l[2], l[3]);
}

template <int TYPE>
__global__ void __launch_bounds__(TI_THREADS, 1)
gemm_i8_tcgen05_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *dst, int64_t lddst, int64_t n, int nb, int64_t m, int *err,
                       GroupMap gm) {
    using T = TiTraits<TYPE>;
    constexpr bool Q6 = TYPE == B200_TYPE_Q6_K;
    constexpr int STAGE_BYTES = TiSizes<TYPE>::STAGE_BYTES;
    constexpr int A_BYTES = T::PLANES * TI_PLANE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ TiBars bars;
    __shared__ int col_act_s[TI_COLS], col_out_s[TI_COLS];
    pdl_trigger();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tile0 = (int64_t)blockIdx.y * (TI_ROWS / TILE_ROWS);
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    int64_t col0 = (int64_t)blockIdx.x * TI_COLS;
    const int64_t K = acts.k;
    volatile int *abort_flag = &bars.abort_flag;
    const bool grouped = gm.work_expert != nullptr;
    if (grouped) {
        pdl_wait();   // the work list is a previous kernel's output
        const int e = gm.work_expert[blockIdx.x];
        if (e < 0) return;   // every thread of the CTA: nothing has been allocated yet
        tiles += (int64_t)e * gm.expert_bytes;
        if (threadIdx.x < TI_COLS) {
            col_act_s[threadIdx.x] = gm.col_act[(int64_t)blockIdx.x * TI_COLS + threadIdx.x];
            col_out_s[threadIdx.x] = gm.col_out[(int64_t)blockIdx.x * TI_COLS + threadIdx.x];
        }
        // columns are addressed through the two tables from here on: column c reads activation row col_act_s[c]
        // (the first column's row stands in for unused columns) and writes output row col_out_s[c]
        col0 = 0;
        m = TI_COLS;
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < T::STAGES; i++) {
            mbar_init(smem_u32(&bars.full[i]), TI_PROD_WARPS);
            mbar_init(smem_u32(&bars.empty[i]), 1 + TI_EPI_WARPS);
        }
        for (int i = 0; i < TI_TSTAGES; i++) {
            mbar_init(smem_u32(&bars.tfull[i]), 1);
            mbar_init(smem_u32(&bars.tempty[i]), TI_EPI_WARPS);
        }
        bars.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TI_EPI_WARPS + TI_PROD_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bars.tmem_base;
    if (!grouped) pdl_wait();

    if (warp < TI_EPI_WARPS) {
        // ---- epilogue: the f32 chain of weight row 32 q + lane over 16 activation rows ----
        const int q = warp & 3, h = warp >> 2;
        const int64_t tile = tile0 + q;
        const bool row_ok = tile < tiles_n;
        const bool any_col = col0 + 16 * h < m;
        const uint8_t *chunk0 = tiles + (row_ok ? tile : 0) * (int64_t)nb * T::CHUNK;
        float acc[16];
#pragma unroll
        for (int c = 0; c < 16; c++) acc[c] = 0.0f;
        for (int b = 0; b < nb; b++) {
            const int s = b % T::STAGES, t = b % TI_TSTAGES;
            const uint32_t sph = (uint32_t)(b / T::STAGES) & 1u, tph = (uint32_t)(b / TI_TSTAGES) & 1u;
            // this row's weight scales of the group
            uint4 ws = make_uint4(0, 0, 0, 0);
            if (row_ok) {
                const uint8_t *chunk = chunk0 + (int64_t)b * T::CHUNK;
                if (TYPE == B200_TYPE_Q8_0) ws = *(const uint4 *)(chunk + 8192 + lane * 16);
                else if (TYPE == B200_TYPE_Q4_0) ws = *(const uint4 *)(chunk + 4096 + lane * 16);
                else if (TYPE == B200_TYPE_MXFP4) { const uint2 e = *(const uint2 *)(chunk + 4096 + lane * 8); ws = make_uint4(e.x, e.y, 0, 0); }
                else ws.x = *(const uint16_t *)(chunk + 6656 + lane * 2);
            }
            const bool ready = mbar_wait(smem_u32(&bars.full[s]), sph, abort_flag) && mbar_wait(smem_u32(&bars.tfull[t]), tph, abort_flag);
            if (!__all_sync(0xffffffffu, ready)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float *sc = (const float *)(smem + s * STAGE_BYTES + A_BYTES + TI_B_BYTES);
            const uint32_t trow = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)(t * 256 + 16 * h);
            if (Q6) {
                int hi[16], lo[16];
                tmem_ld16(hi, trow);
                tmem_ld16(lo, trow + (uint32_t)TI_COLS);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars.tempty[t]));
                if (any_col) {
                    const float dw = f16_bits_to_f32((uint16_t)ws.x);
#pragma unroll
                    for (int c = 0; c < 16; c++) {
                        const int s1 = 64 * hi[c] + lo[c];
                        const float r = __fmul_rn(dw, (float)s1);
                        acc[c] = __fmaf_rn(r, sc[16 * h + c], acc[c]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    int d0[16];
                    tmem_ld16(d0, trow + (uint32_t)(j * TI_COLS));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (j == 7) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars.tempty[t]));
                    }
                    if (any_col) {
                        float dw;
                        if (TYPE == B200_TYPE_MXFP4) {
                            const uint32_t e4 = j < 4 ? ws.x : ws.y;
                            dw = e8m0_half_to_f32((e4 >> (8 * (j & 3))) & 0xffu);
                        } else {
                            const uint32_t dpair = j < 2 ? ws.x : j < 4 ? ws.y : j < 6 ? ws.z : ws.w;
                            dw = f16_bits_to_f32((uint16_t)((j & 1) ? dpair >> 16 : dpair & 0xffffu));
                        }
#pragma unroll
                        for (int c = 0; c < 16; c++) acc[c] = __fmaf_rn((float)d0[c], __fmul_rn(dw, sc[j * TI_COLS + 16 * h + c]), acc[c]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.empty[s]));
        }
        const int64_t row = tile * TILE_ROWS + lane;
        if (row_ok && row < n && !*abort_flag) {
#pragma unroll
            for (int c = 0; c < 16; c++) {
                const int64_t col = col0 + 16 * h + c;
                if (grouped) {
                    const int orow = col_out_s[16 * h + c];
                    if (orow >= 0) dst[(int64_t)orow * lddst + row] = acc[c];
                } else if (col < m) {
                    dst[col * lddst + row] = acc[c];
                }
            }
        }
    } else if (warp < TI_EPI_WARPS + TI_PROD_WARPS) {
        // ---- producers: thread p owns weight row p of the CTA ----
        const int pw = warp - TI_EPI_WARPS, p = pw * 32 + lane;
        const int64_t tile = tile0 + pw;
        const bool tile_ok = tile < tiles_n;
        const uint8_t *wsrc = tiles + (tile_ok ? tile : 0) * (int64_t)nb * T::CHUNK + lane * 16;
        const uint32_t a_off = (uint32_t)((p >> 3) * 2048 + (p & 7) * 16);
        // activation blocks: four 16-byte pieces per thread, consecutive lanes on consecutive columns
        int64_t bcol[4];
        uint32_t b_off[4];
#pragma unroll
        auto act_row = [&](int col) -> int64_t {
            if (grouped) {
                const int r = col_act_s[col];
                return r >= 0 ? r : col_act_s[0];
            }
            const int64_t c = col0 + col;
            return c < m ? c : m - 1;
        };
        for (int j = 0; j < 4; j++) {
            const int i = p + 128 * j, col = i & 31, kc = i >> 5;
            bcol[j] = act_row(col) * K + kc * 16;
            b_off[j] = (uint32_t)((col >> 3) * 2048 + kc * 128 + (col & 7) * 16);
        }
        // activation scales: 32-element types: 8 blocks x 32 columns, two per thread; Q6_K: 32 columns (warp 0 of the producers)
        const int sblk = p >> 4, scol2 = (p & 15) * 2;
        const int64_t sc0 = act_row(scol2), sc1 = act_row(scol2 + 1);
        const int64_t dcol = act_row(lane);
        constexpr int NQ = TYPE == B200_TYPE_Q8_0 ? 16 : TYPE == B200_TYPE_Q6_K ? 13 : 8;   // 16-byte pieces of the row's group
        for (int b = 0; b < nb; b++) {
            const int s = b % T::STAGES;
            const uint32_t sph = (uint32_t)(b / T::STAGES) & 1u;
            uint4 w[NQ], y[4];
            const uint8_t *chunk = wsrc + (int64_t)b * T::CHUNK;
#pragma unroll
            for (int c = 0; c < NQ; c++) w[c] = tile_ok ? ld_stream16(chunk + c * 512) : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int j = 0; j < 4; j++) y[j] = *(const uint4 *)(acts.qs + bcol[j] + (int64_t)b * 256);
            float s0v = 0.0f, s1v = 0.0f;
            if (Q6) {
                if (pw == 0) s0v = acts.d[dcol * nb + b];
            } else {
                s0v = f16_bits_to_f32(acts.dh[sc0 * (K / 32) + (int64_t)b * 8 + sblk]);
                s1v = f16_bits_to_f32(acts.dh[sc1 * (K / 32) + (int64_t)b * 8 + sblk]);
            }
            if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.empty[s]), sph ^ 1u, abort_flag))) break;
            uint8_t *stage = smem + s * STAGE_BYTES;
            uint8_t *A = stage + a_off, *B = stage + A_BYTES;
            if (TYPE == B200_TYPE_Q8_0) {
#pragma unroll
                for (int c = 0; c < 16; c++) *(uint4 *)(A + c * 128) = w[c];   // piece c = elements 16 c .. 16 c + 15
            } else if (TYPE == B200_TYPE_Q4_0 || TYPE == B200_TYPE_MXFP4) {
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    // piece c = block c: low nibbles = elements 0..15 of the block, high nibbles = elements 16..31
                    uint4 lo, hi;
                    lo.x = w[c].x & 0x0f0f0f0fu; lo.y = w[c].y & 0x0f0f0f0fu; lo.z = w[c].z & 0x0f0f0f0fu; lo.w = w[c].w & 0x0f0f0f0fu;
                    hi.x = (w[c].x >> 4) & 0x0f0f0f0fu; hi.y = (w[c].y >> 4) & 0x0f0f0f0fu;
                    hi.z = (w[c].z >> 4) & 0x0f0f0f0fu; hi.w = (w[c].w >> 4) & 0x0f0f0f0fu;
                    if (TYPE == B200_TYPE_MXFP4) {
                        lo.x = mxfp4_lut4(lo.x); lo.y = mxfp4_lut4(lo.y); lo.z = mxfp4_lut4(lo.z); lo.w = mxfp4_lut4(lo.w);
                        hi.x = mxfp4_lut4(hi.x); hi.y = mxfp4_lut4(hi.y); hi.z = mxfp4_lut4(hi.z); hi.w = mxfp4_lut4(hi.w);
                    } else {
                        lo.x = nibbles_minus8(lo.x); lo.y = nibbles_minus8(lo.y); lo.z = nibbles_minus8(lo.z); lo.w = nibbles_minus8(lo.w);
                        hi.x = nibbles_minus8(hi.x); hi.y = nibbles_minus8(hi.y); hi.z = nibbles_minus8(hi.z); hi.w = nibbles_minus8(hi.w);
                    }
                    *(uint4 *)(A + (2 * c) * 128) = lo;
                    *(uint4 *)(A + (2 * c + 1) * 128) = hi;
                }
            } else {
                // Q6_K: ql pieces 0..7, qh pieces 8..11, the 16 scales in piece 12 (crates/ggml/src/quants.rs:585-612)
                const uint4 scv = w[12];
                const uint32_t scw[4] = {scv.x, scv.y, scv.z, scv.w};
#pragma unroll
                for (int nn = 0; nn < 2; nn++)
#pragma unroll
                    for (int l16 = 0; l16 < 2; l16++) {
                        const uint4 a = w[4 * nn + l16], bq = w[4 * nn + 2 + l16], hq = w[8 + 2 * nn + l16];
                        uint4 v[4];
                        v[0] = make_uint4((a.x & 0x0f0f0f0fu) | ((hq.x << 4) & 0x30303030u), (a.y & 0x0f0f0f0fu) | ((hq.y << 4) & 0x30303030u),
                                          (a.z & 0x0f0f0f0fu) | ((hq.z << 4) & 0x30303030u), (a.w & 0x0f0f0f0fu) | ((hq.w << 4) & 0x30303030u));
                        v[1] = make_uint4((bq.x & 0x0f0f0f0fu) | ((hq.x << 2) & 0x30303030u), (bq.y & 0x0f0f0f0fu) | ((hq.y << 2) & 0x30303030u),
                                          (bq.z & 0x0f0f0f0fu) | ((hq.z << 2) & 0x30303030u), (bq.w & 0x0f0f0f0fu) | ((hq.w << 2) & 0x30303030u));
                        v[2] = make_uint4(((a.x >> 4) & 0x0f0f0f0fu) | (hq.x & 0x30303030u), ((a.y >> 4) & 0x0f0f0f0fu) | (hq.y & 0x30303030u),
                                          ((a.z >> 4) & 0x0f0f0f0fu) | (hq.z & 0x30303030u), ((a.w >> 4) & 0x0f0f0f0fu) | (hq.w & 0x30303030u));
                        v[3] = make_uint4(((bq.x >> 4) & 0x0f0f0f0fu) | ((hq.x >> 2) & 0x30303030u), ((bq.y >> 4) & 0x0f0f0f0fu) | ((hq.y >> 2) & 0x30303030u),
                                          ((bq.z >> 4) & 0x0f0f0f0fu) | ((hq.z >> 2) & 0x30303030u), ((bq.w >> 4) & 0x0f0f0f0fu) | ((hq.w >> 2) & 0x30303030u));
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int kc = 8 * nn + 2 * e + l16;   // the 16-element run and its scale
                            const int scale = (int)(int8_t)(scw[kc >> 2] >> (8 * (kc & 3)));
                            uint4 hi, lo;
                            q6_planes(v[e], scale, &hi, &lo);
                            *(uint4 *)(A + kc * 128) = hi;
                            *(uint4 *)(A + TI_PLANE_BYTES + kc * 128) = lo;
                        }
                    }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) *(uint4 *)(B + b_off[j]) = y[j];
            float *sc = (float *)(stage + A_BYTES + TI_B_BYTES);
            if (Q6) {
                if (pw == 0) sc[lane] = s0v;
            } else {
                sc[sblk * TI_COLS + scol2] = s0v;
                sc[sblk * TI_COLS + scol2 + 1] = s1v;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.full[s]));
        }
    } else if (lane == 0) {
        // ---- MMA issue ----
        for (int b = 0; b < nb; b++) {
            const int s = b % T::STAGES, t = b % TI_TSTAGES;
            const uint32_t sph = (uint32_t)(b / T::STAGES) & 1u, tph = (uint32_t)(b / TI_TSTAGES) & 1u;
            if (!mbar_wait(smem_u32(&bars.full[s]), sph, abort_flag)) break;
            if (!mbar_wait(smem_u32(&bars.tempty[t]), tph ^ 1u, abort_flag)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_base = smem_u32(smem + s * STAGE_BYTES), b_base = a_base + A_BYTES;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint64_t bdesc = smem_desc(b_base + j * 256);
                if (Q6) {
                    // block j of the hi plane accumulates into columns 0..31, of the lo plane into 32..63
                    const uint32_t accumulate = j == 0 ? 0u : 1u;
                    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(
                                     tmem + (uint32_t)(t * 256)),
                                 "l"(smem_desc(a_base + j * 256)), "l"(bdesc), "r"(TI_IDESC), "r"(accumulate)
                                 : "memory");
                    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(
                                     tmem + (uint32_t)(t * 256 + TI_COLS)),
                                 "l"(smem_desc(a_base + TI_PLANE_BYTES + j * 256)), "l"(bdesc), "r"(TI_IDESC), "r"(accumulate)
                                 : "memory");
                } else {
                    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p; }" ::"r"(
                                     tmem + (uint32_t)(t * 256 + j * TI_COLS)),
                                 "l"(smem_desc(a_base + j * 256)), "l"(bdesc), "r"(TI_IDESC), "r"(0)
                                 : "memory");
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.empty[s])) : "memory");
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars.tfull[t])) : "memory");
        }
    }
    // ---- teardown: every role has left its loop (finished, or gave up) ----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TI_EPI_WARPS + TI_PROD_WARPS) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && bars.abort_flag) atomicExch(err, TI_ERR_WAIT);
}

template <int TYPE>
int launch_i8(int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst, cudaStream_t s,
              GroupMap gm = GroupMap{nullptr, nullptr, nullptr, 0}, int64_t work_items = 0) {
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_i8_tcgen05_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, TiSizes<TYPE>::SMEM_BYTES));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const int nb = (int)(k / GROUP_K);
    const int64_t gx = gm.work_expert ? work_items : (m + TI_COLS - 1) / TI_COLS, gy = (n + TI_ROWS - 1) / TI_ROWS;
    B200_REQUIRE(gx < 0x7fffffffLL && gy <= 65535, "gemm: %lld x %lld is too large for one launch", (long long)n, (long long)m);
    return launch_pdl(gemm_i8_tcgen05_kernel<TYPE>, dim3((unsigned)gx, (unsigned)gy), dim3(TI_THREADS), (size_t)TiSizes<TYPE>::SMEM_BYTES, s, tiles, acts,
                      dst, lddst, n, nb, m, err, gm);
}

// ---- MUL_MAT_ID: (token, slot) pairs grouped by expert ---------------------------------------------------------
// counts[e] = pairs routed to expert e (the ids outside [0, n_expert) are skipped, as the per-pair kernels skip them)
__global__ void mmid_count_kernel(const int32_t *ids, int n_pairs, int n_expert, int *counts) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = ids[i];
    if (e >= 0 && e < n_expert) atomicAdd(&counts[e], 1);
}
// one CTA: work items per expert (32 pairs each) laid out expert after expert; first_item[e] = the expert's first item
__global__ void mmid_plan_kernel(const int *counts, int n_expert, int max_items, int *first_item, int *cursor, int *work_expert, int *col_act,
                                 int *col_out) {
    pdl_trigger();
    pdl_wait();
    __shared__ int total;
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < n_expert; e++) {
            first_item[e] = at;
            cursor[e] = 0;
            const int items = (counts[e] + TI_COLS - 1) / TI_COLS;
            for (int i = 0; i < items && at + i < max_items; i++) work_expert[at + i] = e;
            at += items;
        }
        total = at < max_items ? at : max_items;
        for (int w = total; w < max_items; w++) work_expert[w] = -1;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < max_items * TI_COLS; i += blockDim.x) {
        col_act[i] = -1;
        col_out[i] = -1;
    }
}
// pair i takes the next free column of its expert's items (the order inside an expert does not matter: every output
// element depends on its own pair only)
__global__ void mmid_scatter_kernel(const int32_t *ids, int n_pairs, int n_ids, int ne11, int n_expert, const int *first_item, int *cursor,
                                    int *col_act, int *col_out) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = ids[i];
    if (e < 0 || e >= n_expert) return;
    const int at = atomicAdd(&cursor[e], 1);
    const int tok = i / n_ids, slot = i % n_ids;
    const int64_t col = (int64_t)first_item[e] * TI_COLS + at;
    col_act[col] = tok * ne11 + slot % ne11;   // crates/ggml/src/compute.rs:2124: the activation row of a slot
    col_out[col] = i;
}

}  // namespace

// MUL_MAT_ID over MXFP4 / Q4_0 experts whose row count takes the 8x8 route (the chain of the per-pair gemv,
// crates/ggml/src/compute.rs:2131-2151, repack.rs:1048-1068, is the per-block fma of this kernel): the pairs are counted
// and grouped by expert on the device, and every expert's weights meet all the rows routed to it in tensor-core tiles
// of 32 pairs.  lists: scratch of mmid_grouped_scratch_bytes(n_expert, pairs) bytes.
size_t mmid_grouped_scratch_bytes(int64_t n_expert, int64_t n_pairs) {
    const int64_t max_items = n_pairs / TI_COLS + n_expert;
    return (size_t)(3 * n_expert + max_items + 2 * max_items * TI_COLS) * sizeof(int) + 256;
}
int launch_mul_mat_id_grouped(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok, int64_t n_ids, const uint8_t *tiles,
                              ActView acts, const int32_t *ids, float *dst, void *lists, cudaStream_t s) {
    B200_REQUIRE(type == B200_TYPE_MXFP4 || type == B200_TYPE_Q4_0, "mul_mat_id grouped: type %d is not a 32-element-block type on the 8x8 route", type);
    const int64_t n_pairs = n_tok * n_ids;
    B200_REQUIRE(n_pairs < 0x7fffffffLL / TI_COLS && n_expert < (1 << 20), "mul_mat_id grouped: too many pairs or experts");
    const int64_t max_items = n_pairs / TI_COLS + n_expert;
    int *counts = (int *)lists, *first_item = counts + n_expert, *cursor = first_item + n_expert, *work_expert = cursor + n_expert;
    int *col_act = work_expert + max_items, *col_out = col_act + max_items * TI_COLS;
    B200_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)n_expert, s));
    int rc = launch_pdl(mmid_count_kernel, dim3((unsigned)((n_pairs + 255) / 256)), dim3(256), 0, s, ids, (int)n_pairs, (int)n_expert, counts);
    if (rc != B200_STATUS_SUCCESS) return rc;
    rc = launch_pdl(mmid_plan_kernel, dim3(1), dim3(256), 0, s, (const int *)counts, (int)n_expert, (int)max_items, first_item, cursor, work_expert,
                    col_act, col_out);
    if (rc != B200_STATUS_SUCCESS) return rc;
    rc = launch_pdl(mmid_scatter_kernel, dim3((unsigned)((n_pairs + 255) / 256)), dim3(256), 0, s, ids, (int)n_pairs, (int)n_ids, (int)ne11, (int)n_expert,
                    (const int *)first_item, cursor, col_act, col_out);
    if (rc != B200_STATUS_SUCCESS) return rc;
    GroupMap gm;
    gm.work_expert = work_expert;
    gm.col_act = col_act;
    gm.col_out = col_out;
    gm.expert_bytes = (int64_t)((n + TILE_ROWS - 1) / TILE_ROWS) * (k / GROUP_K) * chunk_bytes(type);
    if (type == B200_TYPE_MXFP4) return launch_i8<B200_TYPE_MXFP4>(n, k, TI_COLS, tiles, acts, dst, n, s, gm, max_items);
    return launch_i8<B200_TYPE_Q4_0>(n, k, TI_COLS, tiles, acts, dst, n, s, gm, max_items);
}

// Q8_0 (fast numerics), Q4_0, MXFP4 (8x8 gemm chain) and Q6_K (tiled chain) prompt mat-muls, 32 activation rows and up
int launch_gemm_tcgen05_i8(int type, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                           cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemm: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    switch (type) {
        case B200_TYPE_Q8_0: return launch_i8<B200_TYPE_Q8_0>(n, k, m, tiles, acts, dst, lddst, s);
        case B200_TYPE_Q4_0: return launch_i8<B200_TYPE_Q4_0>(n, k, m, tiles, acts, dst, lddst, s);
        case B200_TYPE_MXFP4: return launch_i8<B200_TYPE_MXFP4>(n, k, m, tiles, acts, dst, lddst, s);
        case B200_TYPE_Q6_K: return launch_i8<B200_TYPE_Q6_K>(n, k, m, tiles, acts, dst, lddst, s);
        default: B200_REQUIRE(false, "gemm: no int8 tensor-core kernel for weight type %d", type);
    }
}

}  // namespace b200
