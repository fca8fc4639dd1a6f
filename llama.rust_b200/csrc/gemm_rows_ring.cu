// Q4_K mat-mul over a handful of activation rows (a batched decode step: 8 to 31), persistent form.
//
// The few-rows kernel of gemm_mma.cu gives a CTA one 32-row tile and has its warps take two phases in step (integer
// dots of a window of super-blocks, then the f32 chain over the window), so a launch costs windows x waves of a
// phase pair whatever the bytes.  Here one CTA per SM walks its share of the row tiles, and three kinds of warps
// work on different super-blocks at the same time, handing slots of two rings to one another through mbarriers:
//   * eight producer lanes bring units = (row tile, super-block), 4608 weight bytes each, into the slots of the weight
//     ring, one bulk copy per unit;
//   * eight multiply warps take units round-robin: the unit's activations as whole 16-byte pieces from global memory (L2
//     hits, asked for before the wait for the slot) through a staging area of the warp's own into fragments, weight
//     fragments from the slot into registers (the slot goes back to the producers at once), one mma.sync (m16n8k32,
//     s8 x s8 -> s32, accumulator cleared) per sub-block and 16 x 8 patch, the 6-bit scales applied as integers, and the
//     scaled pair dots into the warp's slot of the second ring together with the rows' unpacked headers and the columns'
//     packed sums;
//   * eight chain warps (thread = one row x two columns) take the units in K order and run the 8x8 gemm chain of
//     crates/ggml/src/repack.rs:1692-1768: sumf = fma(f32(ig[g]), d * d_x, sumf), summin = fma(f32(mg[g]), dmin * d_x,
//     summin) for the four sub-block pairs, out = sumf - summin after the tile's last super-block.
// Measured on the way (4096 x 14336 x 16, SM clocks per unit of one CTA): the activations as 32 more small bulk copies
// per unit 2700; one producer lane for all units 860, of which 500 to 900 behind each bulk-copy instruction whatever its
// size, hence eight issuing lanes; nine 16-byte cp.async copies per lane of a producer warp instead: the multiply warps'
// activation loads then took 960 cycles per unit to issue behind the outstanding misses; 8-byte activation fragment
// loads straight from global memory touch 128 lines per unit, the 16-byte pieces 32.  As it stands a unit costs about
// 700 cycles (a multiply warp 4700 per unit of its own, 2000 of them waiting; the chain 330), against 740 for the
// per-tile kernel.
// The arithmetic, and so every bit of the result, is that of gemm_q4_K_small_kernel and of the CPU.
//
// Every wait is bounded: a wait that runs out records error code 4 in the device's error word, raises the CTA's
// abort flag, the roles leave their loops without storing, and the producer lanes wait (bounded again) for the copies
// they still have in flight before the CTA ends.
#include <cstdlib>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int RR_WSLOTS = 24;                  // weight ring: a slot is in use from the copy's issue (a trip to HBM of 3 us under load) until a multiply warp has it in registers
constexpr int RR_OSLOTS = 8;                   // ring of scaled dots: one slot per multiply warp
constexpr int RR_ISSUERS = 8;                   // producer lanes; divides RR_WSLOTS, so a slot always has the same issuer
constexpr int RR_XPITCH = 288;                 // a staged activation row: 256 bytes plus 32, so that the eight columns of a fragment load fall in different banks
constexpr int RR_MUL_WARPS = 8, RR_CHAIN_WARPS = 8;
constexpr int RR_THREADS = 128 + RR_MUL_WARPS * 32 + RR_CHAIN_WARPS * 32;   // warp group 0: four producer warps
constexpr unsigned RR_SPIN_LIMIT = 1u << 20;   // polls with a short sleep between them: about a second in all
constexpr int RR_ERR_WAIT = 4;                 // device error word: a pipeline wait ran out

// what a multiply warp leaves for the chain warps
struct RrSlot {
    int4 ig[16][33];                           // [column][row] = the four scaled pair dots
    uint4 hdr[32];                             // row r: d, dmin as f32 bits, mins 0..3, mins 4..7 one per byte
    uint4 bp[16];                              // column c: the eight sub-block sums, two per word
    uint2 sc[32];                              // row r: the eight 6-bit scales one per byte
    float da[16];                              // column c: the super-block's activation scale
};
static_assert(sizeof(RrSlot) % 16 == 0, "slots keep their 16-byte alignment");

struct RrMats {
    const uint8_t *tiles[3];
    float *dst[3];
    int64_t n[3], lddst[3];
    int tile_start[4];                         // matrix e owns row tiles tile_start[e] .. tile_start[e + 1] of the launch
};

// two rings: the weights (producer -> multiply warps; a slot is free again as soon as its unit is in the multiply warp's
// registers) and the scaled dots (multiply warps -> chain warps)
struct RrShared {
    uint8_t w[RR_WSLOTS][4608];                // a unit: 32 row headers, then 8 pieces of 32 rows x 16 bytes
    RrSlot slot[RR_OSLOTS];
    int8_t xs[RR_MUL_WARPS][16 * RR_XPITCH];   // a multiply warp's staging of its unit's activations: column c's 256 values at c * RR_XPITCH
    uint64_t full[RR_WSLOTS], wfree[RR_WSLOTS], done[RR_OSLOTS], empty[RR_OSLOTS];
    int abort_flag;
};

__device__ __forceinline__ uint32_t rr_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void rr_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(rr_smem(bar)), "r"(count));
}
__device__ __forceinline__ void rr_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(rr_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void rr_bulk(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(rr_smem(dst_smem)), "l"(src_gmem),
                 "r"(bytes), "r"(rr_smem(bar))
                 : "memory");
}
__device__ __forceinline__ void rr_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(rr_smem(bar)) : "memory");
}
// bounded wait for the phase with the given parity; false on expiry or when the CTA is winding down
__device__ __forceinline__ bool rr_wait(uint64_t *bar, unsigned parity, unsigned limit, const int *abort_flag) {
    const uint32_t a = rr_smem(bar);
    for (unsigned i = 0; i < limit; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"   // suspended for up to the hinted time, woken by the phase
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity), "r"(1000u)
            : "memory");
        if (ok) return true;
        if (*(volatile const int *)abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void rr_mma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// c + (low half of a) * (byte 0 of b) + (high half of a) * (byte 1 of b), halves signed, bytes unsigned; _hi: bytes 2 and 3
__device__ __forceinline__ int rr_dp2a_lo(uint32_t a, uint32_t b) {
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(0));
    return d;
}
__device__ __forceinline__ int rr_dp2a_hi(uint32_t a, uint32_t b) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(0));
    return d;
}

// the CTA's i-th row tile: which matrix, which tile of it
struct RrTile {
    int me;
    int64_t tile;
};
__device__ __forceinline__ RrTile rr_tile(const RrMats &mats, int64_t i) {
    const int64_t g = (int64_t)blockIdx.x + i * gridDim.x;
    RrTile t;
    t.me = g >= mats.tile_start[2] ? 2 : g >= mats.tile_start[1] ? 1 : 0;
    t.tile = g - mats.tile_start[t.me];
    return t;
}

__global__ void __launch_bounds__(RR_THREADS, 1)
gemm_q4_K_rows_ring_kernel(const RrMats mats, ActView acts, int nb, int64_t m, int *err, unsigned spin_limit, int skip_unit) {
    extern __shared__ __align__(128) unsigned char rr_raw[];
    RrShared &sh = *(RrShared *)rr_raw;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int total_tiles = mats.tile_start[3];
    const int my_tiles = (int)blockIdx.x < total_tiles ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int units = my_tiles * nb;   // the launcher keeps this below 2^31
    const int64_t col0 = (int64_t)blockIdx.y * 16;
    const int64_t K = acts.k;

    if (tid == 0) {
        for (int i = 0; i < RR_WSLOTS; i++) {
            rr_init(&sh.full[i], 1);
            rr_init(&sh.wfree[i], 1);
        }
        for (int i = 0; i < RR_OSLOTS; i++) {
            rr_init(&sh.done[i], 1);
            rr_init(&sh.empty[i], RR_CHAIN_WARPS);
        }
        sh.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    unsigned issued_mask = 0, issued_parity = 0;   // a producer lane's record of the copies it started: slots used, parity of the last phase on each

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        {
            // ---------------- producer lanes (four of each warp; unit u goes to issuer u % 16, which owns that ring slot): the
            // weights do not depend on the previous kernel in the stream.  One bulk copy per unit.  A bulk-copy instruction holds
            // its lane for 500 to 900 cycles whatever its size, hence many issuing lanes; nine 16-byte cp.async copies per lane of
            // a warp instead kept so many L1 misses outstanding that the multiply warps' activation loads (L2 hits) waited 960
            // cycles per unit to issue.
            if (lane < 2) {   // issuer q = 2 warp + lane: units q, q + 8, .., ring slots q, q + 8 and q + 16 in turn
                for (int u = 2 * warp + lane; u < units; u += RR_ISSUERS) {
                    const int st = u % RR_WSLOTS;
                    const unsigned ph = (unsigned)((u / RR_WSLOTS) & 1);
                    const int ti = u / nb;
                    const int b = u - ti * nb;
                    if (u >= RR_WSLOTS && !rr_wait(&sh.wfree[st], ph ^ 1, spin_limit, &sh.abort_flag)) {
                        if (!*(volatile int *)&sh.abort_flag) {
                            atomicExch(err, RR_ERR_WAIT);
                            *(volatile int *)&sh.abort_flag = 1;
                        }
                        break;
                    }
                    if (*(volatile int *)&sh.abort_flag) break;
                    if (!(blockIdx.x == 0 && blockIdx.y == 0 && u == skip_unit)) {   // skip_unit >= 0 only in the wait-expiry test: that slot is never filled
                        const RrTile cur = rr_tile(mats, ti);
                        rr_expect_tx(&sh.full[st], 4608);
                        rr_bulk(sh.w[st], mats.tiles[cur.me] + (cur.tile * nb + b) * (int64_t)4608, 4608, &sh.full[st]);
                        issued_mask |= 1u << st;
                        issued_parity = (issued_parity & ~(1u << st)) | (ph << st);
                    }
                }
            }
        }
    } else if (warp < 4 + RR_MUL_WARPS) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
        // ---------------- multiply warps: unit u goes to warp u % 8, which so sees every phase of the weight slots it reads
        const int mw = warp - 4;
        const int g8 = lane >> 2, t = lane & 3;
        pdl_wait();   // the activations come from the previous kernel in the stream
        // the unit's activations come as whole 16-byte pieces (lane = piece lane % 16 of column 2 i + lane / 16: four full lines per
        // load instruction; 8-byte fragment loads straight from global memory touched 128 lines per unit) into the warp's staging
        // rows, and from there as fragments; sums: two items of 16 columns x 4 sub-block pairs.  Columns clamped to the last valid one.
        const int8_t *xbase = acts.qs + 16 * (lane & 15);
        const int64_t ccol = col0 + (lane >> 4), clast = m - 1;
        int8_t *xst = sh.xs[mw];
        const int16_t *scol[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int i = lane + 32 * j;
            const int64_t cs = col0 + (i >> 2) < m ? col0 + (i >> 2) : m - 1;
            scol[j] = acts.bsums + cs * (K / 16) + 4 * (i & 3);
        }
        const float *dcol = acts.d + (col0 + (lane & 15) < m ? col0 + (lane & 15) : m - 1) * nb;
        for (int u = mw; u < units; u += RR_MUL_WARPS) {
            const int st = u % RR_WSLOTS;
            const unsigned ph = (unsigned)((u / RR_WSLOTS) & 1);
            const int os = u % RR_OSLOTS;                                // = mw: a multiply warp has one slot of scaled dots
            const unsigned oph = (unsigned)((u / RR_OSLOTS) & 1);
            const int b = u % nb;
            // the unit's activations, sums and scales: asked for before the wait for the slot
            uint4 xa[8];
            short4 s4[2];
#pragma unroll
            for (int i = 0; i < 8; i++) xa[i] = *(const uint4 *)(xbase + (ccol + 2 * i < clast ? ccol + 2 * i : clast) * K + (int64_t)b * 256);
#pragma unroll
            for (int j = 0; j < 2; j++) s4[j] = *(const short4 *)(scol[j] + (int64_t)b * 16);
            const float da_u = dcol[b];
            if (!rr_wait(&sh.full[st], ph, spin_limit, &sh.abort_flag)) {
                if (!*(volatile int *)&sh.abort_flag) {
                    atomicExch(err, RR_ERR_WAIT);
                    *(volatile int *)&sh.abort_flag = 1;
                }
                break;
            }
            // the activations through the staging rows into fragments
            uint2 ya[4][2][2];
#pragma unroll
            for (int i = 0; i < 8; i++) *(uint4 *)(xst + (2 * i + (lane >> 4)) * RR_XPITCH + 16 * (lane & 15)) = xa[i];
            __syncwarp();
#pragma unroll
            for (int g = 0; g < 4; g++)
#pragma unroll
                for (int nt = 0; nt < 2; nt++) {
                    const int8_t *aq = xst + (8 * nt + g8) * RR_XPITCH + 64 * g + 8 * t;
                    ya[g][nt][0] = *(const uint2 *)aq;
                    ya[g][nt][1] = *(const uint2 *)(aq + 32);
                }
            __syncwarp();   // the staging rows are free for the next unit
            // the unit's weights into registers, and its ring slot back to the producers
            const uint8_t *wsm = sh.w[st];
            const uint4 hd = *(const uint4 *)(wsm + lane * 16);
            uint2 wa[2][4], wb[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int ra = 16 * mt + g8, rb = ra + 8;
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const uint8_t *wq = wsm + 512 + (2 * g + (t >> 1)) * 512 + 8 * (t & 1);
                    wa[mt][g] = *(const uint2 *)(wq + ra * 16);
                    wb[mt][g] = *(const uint2 *)(wq + rb * 16);
                }
            }
            __syncwarp();
            if (lane == 0) rr_arrive(&sh.wfree[st]);
            // the slot of the scaled dots: free once the chain warps are through with the unit that had it last
            if (u >= RR_OSLOTS && !rr_wait(&sh.empty[os], oph ^ 1, spin_limit, &sh.abort_flag)) {
                if (!*(volatile int *)&sh.abort_flag) {
                    atomicExch(err, RR_ERR_WAIT);
                    *(volatile int *)&sh.abort_flag = 1;
                }
                break;
            }
            RrSlot &s = sh.slot[os];
            // row `lane`: d, dmin as f32 and the eight 6-bit mins one per byte for the chain threads, the eight 6-bit scales
            // one per byte for this warp's lanes (crates/ggml/src/quants.rs:421-429)
            s.hdr[lane] = make_uint4(__float_as_uint(f16_bits_to_f32((uint16_t)(hd.x & 0xffffu))), __float_as_uint(f16_bits_to_f32((uint16_t)(hd.x >> 16))),
                                     hd.z & 0x3f3f3f3fu, ((hd.w >> 4) & 0x0f0f0f0fu) | (((hd.z >> 6) & 0x03030303u) << 4));
            s.sc[lane] = make_uint2(hd.y & 0x3f3f3f3fu, (hd.w & 0x0f0f0f0fu) | (((hd.y >> 6) & 0x03030303u) << 4));
            if (lane < 16) s.da[lane] = da_u;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int i = lane + 32 * j;
                ((uint32_t *)&s.bp[i >> 2])[i & 3] = (uint32_t)((int)s4[j].x + (int)s4[j].y) & 0xffffu | (uint32_t)((int)s4[j].z + (int)s4[j].w) << 16;
            }
            __syncwarp();
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                const int ra = 16 * mt + g8, rb = ra + 8;
                const uint2 sca = s.sc[ra], scb = s.sc[rb];
                const uint32_t sc[2][2] = {{sca.x, sca.y}, {scb.x, scb.y}};   // [row a / b][sub-blocks 0..3 / 4..7]
                int v[2][4][4];   // [column patch][accumulator][pair]
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    const uint2 va = wa[mt][g], vb = wb[mt][g];
                    const int shf = 16 * (g & 1);
                    int s_lo[2], s_hi[2];
#pragma unroll
                    for (int r = 0; r < 2; r++) {
                        s_lo[r] = (sc[r][g >> 1] >> shf) & 0xff;
                        s_hi[r] = (sc[r][g >> 1] >> (shf + 8)) & 0xff;
                    }
#pragma unroll
                    for (int nt = 0; nt < 2; nt++) {
                        const uint2 y0 = ya[g][nt][0], y1 = ya[g][nt][1];
                        int d0[4], d1[4];
                        rr_mma(d0, va.x & 0x0f0f0f0fu, vb.x & 0x0f0f0f0fu, va.y & 0x0f0f0f0fu, vb.y & 0x0f0f0f0fu, y0.x, y0.y);
                        rr_mma(d1, (va.x >> 4) & 0x0f0f0f0fu, (vb.x >> 4) & 0x0f0f0f0fu, (va.y >> 4) & 0x0f0f0f0fu, (vb.y >> 4) & 0x0f0f0f0fu, y1.x, y1.y);
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
            __syncwarp();
            if (lane == 0) rr_arrive(&sh.done[os]);
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
        // ---------------- chain warps: row `lane`, columns cw and cw + 8, every unit in K order
        const int cw = warp - 4 - RR_MUL_WARPS;
        pdl_wait();   // writes the result
        bool cvalid[2];
#pragma unroll
        for (int j = 0; j < 2; j++) cvalid[j] = col0 + cw + 8 * j < m;
        float sumf[2] = {0.0f, 0.0f}, summin[2] = {0.0f, 0.0f};
        int st = 0, b = 0;
        unsigned ph = 0;
        int64_t ti = 0;
        RrTile cur = rr_tile(mats, 0);
        for (int u = 0; u < units; u++) {
            if (!rr_wait(&sh.done[st], ph, spin_limit, &sh.abort_flag)) {
                if (!*(volatile int *)&sh.abort_flag) {
                    atomicExch(err, RR_ERR_WAIT);
                    *(volatile int *)&sh.abort_flag = 1;
                }
                break;
            }
            const RrSlot &s = sh.slot[st];
            const uint4 hd = s.hdr[lane];
            const uint32_t mn_lo = hd.z, mn_hi = hd.w;
            const float dw = __uint_as_float(hd.x), dmw = __uint_as_float(hd.y);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int c = cw + 8 * j;
                const float da = s.da[c];
                const float sd = __fmul_rn(dw, da), sm = __fmul_rn(dmw, da);
                const int4 ig = s.ig[c][lane];
                const uint4 bp = s.bp[c];
                // pair g: mins 2g and 2g + 1 times the two sub-blocks' activation sums
                const int mg0 = rr_dp2a_lo(bp.x, mn_lo), mg1 = rr_dp2a_hi(bp.y, mn_lo), mg2 = rr_dp2a_lo(bp.z, mn_hi), mg3 = rr_dp2a_hi(bp.w, mn_hi);
                sumf[j] = __fmaf_rn((float)ig.x, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.y, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.z, sd, sumf[j]);
                sumf[j] = __fmaf_rn((float)ig.w, sd, sumf[j]);
                summin[j] = __fmaf_rn((float)mg0, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg1, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg2, sm, summin[j]);
                summin[j] = __fmaf_rn((float)mg3, sm, summin[j]);
            }
            __syncwarp();
            if (lane == 0) rr_arrive(&sh.empty[st]);
            if (++st == RR_OSLOTS) { st = 0; ph ^= 1; }
            if (++b == nb) {
                const int64_t row = cur.tile * TILE_ROWS + lane;
                float *dst = mats.dst[cur.me];
                const int64_t lddst = mats.lddst[cur.me];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    if (row < mats.n[cur.me] && cvalid[j]) {
                        const int64_t col = col0 + cw + 8 * j;
                        const float v = __fsub_rn(sumf[j], summin[j]);
                        dst[col * lddst + row] = v;
                        if (acts.sum) acts.sum[col * acts.ld_sum + row] = __fadd_rn(v, acts.addend[col * acts.ld_addend + row]);
                    }
                    sumf[j] = summin[j] = 0.0f;
                }
                b = 0;
                cur = rr_tile(mats, ++ti);
            }
        }
    }
    // wind-down: every bulk copy this CTA started must have landed before its shared memory is released.  On the normal
    // path the multiply warps have waited for each of them; after an abort the producer lanes wait (bounded) for the last
    // phase they started on each of their slots.
    __syncthreads();
    if (*(volatile int *)&sh.abort_flag && warp < 4 && lane < 2) {
        int never = 0;
        for (int i = 0; i < RR_WSLOTS; i++)
            if (issued_mask & (1u << i)) rr_wait(&sh.full[i], (issued_parity >> i) & 1u, spin_limit < 4096u ? 4096u : spin_limit, &never);
    }
}

// test hook: while spin_limit > 0 the kernel's waits poll at most spin_limit times and the producer of CTA (0, 0) leaves its
// unit skip_unit unfilled (-1 = none), so that a test can watch a wait run out (the kernel returns, error code 4)
int g_rr_wait_limit_override = 0, g_rr_skip_unit = -1;

// B200_GEMM_ROWS_RING=0 keeps the per-tile few-rows kernel, =2 takes this one only for rows of 32 super-blocks and more or more
// row tiles than two per SM; default: every shape (a 16-sequence 8B step as a replayed graph: 5.05 ms without, 4.86 with the
// rule, 4.76 with every shape) (read per call)
int rows_ring_mode() {
    const char *e = getenv("B200_GEMM_ROWS_RING");
    return e && e[0] == '0' ? 0 : e && e[0] == '2' ? 2 : 1;
}

}  // namespace

void gemm_rows_ring_debug_wait(int spin_limit, int skip_unit) {
    g_rr_wait_limit_override = spin_limit > 0 ? spin_limit : 0;
    g_rr_skip_unit = skip_unit;
}

// count Q4_K matrices (8x8 gemm chain) of row length k against the same 8 to 31 activation rows as one persistent launch;
// -1: not a case for this kernel (switched off, no-scratch mode, unaligned activations), the caller takes the per-tile one
int launch_gemm_rows_ring(int count, const int64_t *n, int64_t k, int64_t m, const uint8_t *const *tiles, ActView acts, float *const *dst,
                          const int64_t *lddst, cudaStream_t s) {
    const int mode = g_rr_wait_limit_override > 0 ? 1 : rows_ring_mode();   // the armed test hook takes this kernel
    if (mode == 0 || no_scratch_mode() || count < 1 || count > 3 || m < 1 || m >= 32 || k % GROUP_K) return -1;
    if ((((uintptr_t)acts.qs | (uintptr_t)acts.bsums) & 15) || (k % 256)) return -1;
    for (int e = 0; e < count; e++)
        if ((uintptr_t)tiles[e] & 15) return -1;
    const int nb = (int)(k / GROUP_K);
    RrMats mats;
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
    B200_REQUIRE(total * (k / GROUP_K) < 0x7fffffffLL, "gemm: %lld row tiles are too many for one launch", (long long)total);
    mats.tile_start[3] = (int)total;
    if (total == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(count == 1 || !acts.sum, "gemm: the fused add goes with a single matrix");
    static int sms[64] = {0};
    static bool attr_done[64] = {false};
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemm: device index %d out of range", dev);
    if (!sms[dev]) B200_CUDA(cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev));
    if (mode == 2 && !(nb >= 32 || total > 2 * (int64_t)sms[dev])) return -1;
    if (!attr_done[dev]) {
        B200_CUDA(cudaFuncSetAttribute(gemm_q4_K_rows_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(RrShared)));
        attr_done[dev] = true;
    }
    int *err = nullptr;
    int rc = device_error_word(&err);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const int sy = (int)((m + 15) / 16);
    int64_t gx = sms[dev] / sy;
    if (gx < 1) gx = 1;
    if (gx > total) gx = total;
    // whole rounds: every CTA the same number of tiles where the count allows it (896 tiles on 148 SMs: 7 rounds of 128)
    const int64_t rounds = (total + gx - 1) / gx;
    gx = (total + rounds - 1) / rounds;
    const dim3 grid((unsigned)gx, (unsigned)sy);
    return launch_pdl(gemm_q4_K_rows_ring_kernel, grid, dim3(RR_THREADS), sizeof(RrShared), s, mats, acts, nb, m, err,
                      g_rr_wait_limit_override > 0 ? (unsigned)g_rr_wait_limit_override : RR_SPIN_LIMIT, g_rr_skip_unit);
}

}  // namespace b200
