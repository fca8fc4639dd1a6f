// Decode-shaped mat-mul (few activation rows): HBM-bound streaming kernels.
//
// One CTA owns one 32-row tile of the weight matrix; lane r of every warp owns
// row r, the warps split the 256-element groups of K between them.  Each lane
// reads its row's bytes of a group with 16-byte loads that are contiguous
// across the warp (512 B per load instruction), does the integer block dots
// with dp4a against the Q8 activations (staged per warp in shared memory and
// read as broadcasts), and leaves the exact int32 partials in shared memory.
// After one barrier the f32 accumulation chains are run in ascending K order,
// exactly as the CPU route does, so the result is bit-identical to it:
//   Q4_K 8x8 gemv   crates/ggml/src/repack.rs:1638-1688 (one fma per super-block
//                   for the scale term and one for the min term, out = acc - accmin)
#include "common.cuh"

namespace b200 {

constexpr int GEMV_MAX_WARPS = 16;

// ---------------------------------------------------------------------------
// Q4_K, route REPACK/gemv.  NCOL activation rows share one pass over the weights.
// Shared memory: per warp staging of one activation group per column, and the
// exchange array xch[col][group][row] = {iacc, imin, d|dmin<<16}.
// ---------------------------------------------------------------------------
struct Q4KStage {
    uint4 q[16];   // 256 activation quants of one group
    int bp[8];     // bsums[2j] + bsums[2j+1]
};

template <int NCOL>
__global__ void __launch_bounds__(GEMV_MAX_WARPS * 32)
gemv_q4_K_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *__restrict__ dst, int64_t lddst, int64_t n,
                 int nb) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    Q4KStage *stage = (Q4KStage *)smem + warp * NCOL;
    int4 *xch = (int4 *)(smem + sizeof(Q4KStage) * nwarps * NCOL);  // [NCOL][nb][32], .w unused
    const int64_t tile = blockIdx.x;
    const uint8_t *base = tiles + tile * (int64_t)nb * 4608;

    for (int b = warp; b < nb; b += nwarps) {
        const uint8_t *chunk = base + (int64_t)b * 4608;
        const uint4 h = ld_stream16(chunk + lane * 16);
        uint4 q[8];
#pragma unroll
        for (int c = 0; c < 8; c++) q[c] = ld_stream16(chunk + 512 + c * 512 + lane * 16);
        // stage this group's activations for every column
#pragma unroll
        for (int col = 0; col < NCOL; col++) {
            if (lane < 16) {
                stage[col].q[lane] = *(const uint4 *)(acts.qs + (int64_t)col * acts.k + (int64_t)b * 256 + lane * 16);
            } else if (lane < 24) {
                const int j = lane - 16;
                const short2 s2 = *(const short2 *)(acts.bsums + (int64_t)col * (acts.k / 16) + (int64_t)b * 16 + 2 * j);
                stage[col].bp[j] = (int)s2.x + (int)s2.y;
            }
        }
        __syncwarp();
        // 6-bit scales and mins: crates/ggml/src/quants.rs:421-429 (get_scale_min_k4)
        const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
        const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu;                                         // scales 0..3
        const uint32_t mn_lo4 = u1 & 0x3f3f3f3fu;                                         // mins   0..3
        const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);    // scales 4..7
        const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);  // mins 4..7
#pragma unroll
        for (int col = 0; col < NCOL; col++) {
            int iacc = 0;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                int dlo = 0, dhi = 0;
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    const uint4 w = q[2 * g + hh];
                    const uint4 alo = stage[col].q[4 * g + hh];      // elements 64g + 16hh ..
                    const uint4 ahi = stage[col].q[4 * g + 2 + hh];  // elements 64g + 32 + 16hh ..
                    dlo = __dp4a((int)(w.x & 0x0f0f0f0fu), (int)alo.x, dlo);
                    dlo = __dp4a((int)(w.y & 0x0f0f0f0fu), (int)alo.y, dlo);
                    dlo = __dp4a((int)(w.z & 0x0f0f0f0fu), (int)alo.z, dlo);
                    dlo = __dp4a((int)(w.w & 0x0f0f0f0fu), (int)alo.w, dlo);
                    dhi = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, dhi);
                    dhi = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, dhi);
                    dhi = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, dhi);
                    dhi = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, dhi);
                }
                const uint32_t s4 = g < 2 ? sc_lo4 : sc_hi4;
                const int s_lo = (s4 >> (16 * (g & 1))) & 0xff;
                const int s_hi = (s4 >> (16 * (g & 1) + 8)) & 0xff;
                iacc += dlo * s_lo + dhi * s_hi;
            }
            int imin = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t m4 = j < 4 ? mn_lo4 : mn_hi4;
                imin += (int)((m4 >> (8 * (j & 3))) & 0xff) * stage[col].bp[j];
            }
            xch[((int64_t)col * nb + b) * 32 + lane] = make_int4(iacc, imin, (int)h.x, 0);
        }
        __syncwarp();
    }
    __syncthreads();
    // accumulation chains, ascending K: threads (col, row)
    for (int t = threadIdx.x; t < NCOL * 32; t += blockDim.x) {
        const int col = t >> 5, r = t & 31;
        const float *dx = acts.d + (int64_t)col * nb;
        float sumf = 0.0f, summin = 0.0f;
        for (int b = 0; b < nb; b++) {
            const int4 v = xch[((int64_t)col * nb + b) * 32 + r];
            const float d = f16_bits_to_f32((uint16_t)((uint32_t)v.z & 0xffffu));
            const float dmin = f16_bits_to_f32((uint16_t)((uint32_t)v.z >> 16));
            const float da = dx[b];
            sumf = __fmaf_rn((float)v.x, __fmul_rn(d, da), sumf);
            summin = __fmaf_rn((float)v.y, __fmul_rn(dmin, da), summin);
        }
        const int64_t row = tile * TILE_ROWS + r;
        if (row < n) dst[(int64_t)col * lddst + row] = __fsub_rn(sumf, summin);
    }
}

static int pick_warps(int nb) {
    // the largest warp count <= 16 that divides the group count keeps every warp equally loaded
    for (int w = GEMV_MAX_WARPS; w >= 8; w--)
        if (nb % w == 0) return w;
    return nb < GEMV_MAX_WARPS ? (nb < 1 ? 1 : nb) : GEMV_MAX_WARPS;
}

template <int NCOL>
static int launch_q4k(int64_t n, int nb, const uint8_t *tiles, ActView acts, float *dst, int64_t lddst,
                      cudaStream_t s) {
    const int nw = pick_warps(nb);
    const size_t smem = sizeof(Q4KStage) * nw * NCOL + sizeof(int4) * (size_t)NCOL * nb * 32;
    B200_REQUIRE(smem <= 200 * 1024, "gemv q4_K: k too large for the shared-memory exchange (%zu bytes)", smem);
    static bool attr_done[4] = {false, false, false, false};
    if (!attr_done[NCOL]) {
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<NCOL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done[NCOL] = true;
    }
    const int64_t tiles_n = (n + TILE_ROWS - 1) / TILE_ROWS;
    gemv_q4_K_kernel<NCOL><<<(unsigned)tiles_n, nw * 32, smem, s>>>(tiles, acts, dst, lddst, n, nb);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

int launch_gemv(int type, int route, int64_t n, int64_t k, int64_t m, const uint8_t *tiles, ActView acts, float *dst,
                int64_t lddst, cudaStream_t s) {
    B200_REQUIRE(k % GROUP_K == 0, "gemv: k = %lld must be a multiple of 256", (long long)k);
    const int nb = (int)(k / GROUP_K);
    if (type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK) {
        // columns are processed in passes of at most 3 (the CPU's gemv only ever sees the m % 4 tail rows)
        for (int64_t c0 = 0; c0 < m; c0 += 3) {
            const int nc = (int)(m - c0 < 3 ? m - c0 : 3);
            ActView a = acts;
            a.qs += c0 * k;
            a.d += c0 * nb;
            a.bsums += c0 * (k / 16);
            float *o = dst + c0 * lddst;
            int rc = nc == 1   ? launch_q4k<1>(n, nb, tiles, a, o, lddst, s)
                     : nc == 2 ? launch_q4k<2>(n, nb, tiles, a, o, lddst, s)
                               : launch_q4k<3>(n, nb, tiles, a, o, lddst, s);
            if (rc != B200_STATUS_SUCCESS) return rc;
        }
        return B200_STATUS_SUCCESS;
    }
    B200_REQUIRE(false, "gemv: no kernel for type %d route %d", type, route);
}

}  // namespace b200
