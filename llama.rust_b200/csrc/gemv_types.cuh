// Per-type pieces of the decode mat-mul kernel (gemv.cu): how one lane loads its
// row's bytes of a 256-element group from the tile layout, turns them into exact
// int32 partial dots against the staged Q8 activations, and how the f32
// accumulation chain of the mirrored CPU route consumes those partials.
//
// Exchange layout per (column, group): NW 32-bit words per row, stored
// word-major ([word][row]) so both the writers (lane = row) and the chain
// threads (lane = row) touch consecutive banks.
#pragma once
#include "common.cuh"

namespace b200 {

// activations of one 256-element group staged in shared memory (one per warp and column)
struct ActStage {
    uint4 q[16];    // 256 int8 quants
    int aux[16];    // Q8_K: the 16 bsums;  Q8_0: the 8 scale halves (f16 bits) then 8 block sums
};

__device__ __forceinline__ int dp4(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int w) {
    return w == 0 ? v.x : w == 1 ? v.y : w == 2 ? v.z : v.w;
}

// ---------------------------------------------------------------------------
// Q6_K, row-dot numerics: crates/ggml/src/vec_dot.rs:990-1032.
// Eight f32 lanes per output (lane L gets elements 4L..4L+3 of every 32-group),
// acc[L] = fma(d_x*d_w, sumi[L], acc[L]) per super-block, then the hsum8 tree.
// ---------------------------------------------------------------------------
struct TraitsQ6K {
    static constexpr int TYPE = B200_TYPE_Q6_K;
    static constexpr int CHUNK = 6720;
    static constexpr int NW = 9;        // 8 lane sums + d
    static constexpr int CHAINS = 8;
    static constexpr bool ACT_Q8K = true;

    struct Regs {
        uint4 ql[8], qh[4], sc;
        uint32_t d;
    };
    __device__ static __forceinline__ void load(const uint8_t *chunk, int lane, Regs &r) {
#pragma unroll
        for (int c = 0; c < 8; c++) r.ql[c] = ld_stream16(chunk + c * 512 + lane * 16);
#pragma unroll
        for (int c = 0; c < 4; c++) r.qh[c] = ld_stream16(chunk + 4096 + c * 512 + lane * 16);
        r.sc = ld_stream16(chunk + 6144 + lane * 16);
        r.d = *(const uint16_t *)(chunk + 6656 + lane * 2);
    }
    __device__ static __forceinline__ int scale_at(const uint4 &sc, int b) {
        return (int)(int8_t)(word_of(sc, b >> 2) >> (8 * (b & 3)));
    }
    __device__ static __forceinline__ void compute(const Regs &r, const ActStage &a, uint32_t *xw /* [NW][32] + lane */) {
        int sumi[8];
#pragma unroll
        for (int l = 0; l < 8; l++) sumi[l] = 0;
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
            for (int l16 = 0; l16 < 2; l16++) {
                const uint4 A = r.ql[4 * n + l16], B = r.ql[4 * n + 2 + l16], H = r.qh[2 * n + l16];
                const uint4 y0 = a.q[8 * n + 0 + l16], y1 = a.q[8 * n + 2 + l16];
                const uint4 y2 = a.q[8 * n + 4 + l16], y3 = a.q[8 * n + 6 + l16];
                const int s0 = scale_at(r.sc, 8 * n + 0 + l16), s1 = scale_at(r.sc, 8 * n + 2 + l16);
                const int s2 = scale_at(r.sc, 8 * n + 4 + l16), s3 = scale_at(r.sc, 8 * n + 6 + l16);
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t aw = word_of(A, w), bw = word_of(B, w), hw = word_of(H, w);
                    const uint32_t v0 = (aw & 0x0f0f0f0fu) | ((hw << 4) & 0x30303030u);
                    const uint32_t v1 = (bw & 0x0f0f0f0fu) | ((hw << 2) & 0x30303030u);
                    const uint32_t v2 = ((aw >> 4) & 0x0f0f0f0fu) | (hw & 0x30303030u);
                    const uint32_t v3 = ((bw >> 4) & 0x0f0f0f0fu) | ((hw >> 2) & 0x30303030u);
                    int acc = sumi[4 * l16 + w];
                    acc += s0 * dp4(v0, word_of(y0, w), 0);
                    acc += s1 * dp4(v1, word_of(y1, w), 0);
                    acc += s2 * dp4(v2, word_of(y2, w), 0);
                    acc += s3 * dp4(v3, word_of(y3, w), 0);
                    sumi[4 * l16 + w] = acc;
                }
            }
#pragma unroll
        for (int l = 0; l < 8; l++) {
            // the -32 bias, removed once per lane with the CPU's pairing of bsums and scales
            const int sub = (a.aux[2 * l] * scale_at(r.sc, 2 * l) + a.aux[2 * l + 1] * scale_at(r.sc, 2 * l + 1)) * 32;
            xw[l * 32] = (uint32_t)(sumi[l] - sub);
        }
        xw[8 * 32] = r.d;
    }
    // chain thread (row, l): one fma per super-block
    __device__ static __forceinline__ void chain(float &acc, const uint32_t *xg /* [NW][32] + row */, int l,
                                                 const ActView &acts, int64_t col, int64_t group) {
        const float dx = acts.d[col * (acts.k / 256) + group];
        const float dw = f16_bits_to_f32((uint16_t)xg[8 * 32]);
        acc = __fmaf_rn(__fmul_rn(dx, dw), (float)(int)xg[l * 32], acc);
    }
};

// ---------------------------------------------------------------------------
// Q8_0, row-dot numerics: crates/ggml/src/vec_dot.rs:732-752 (tinyBLAS gives the
// same values, tinyblas.rs:64-74).  acc[L] = fma(d_w*d_x, dot4_L, acc[L]) per
// 32-block, hsum8 at the end.
// ---------------------------------------------------------------------------
struct TraitsQ8_0 {
    static constexpr int TYPE = B200_TYPE_Q8_0;
    static constexpr int CHUNK = 8704;
    static constexpr int NW = 68;       // 8 blocks x 8 lane dots + 4 words of scale halves
    static constexpr int CHAINS = 8;
    static constexpr bool ACT_Q8K = false;

    struct Regs {
        uint4 qs[16], d;
    };
    __device__ static __forceinline__ void load(const uint8_t *chunk, int lane, Regs &r) {
#pragma unroll
        for (int c = 0; c < 16; c++) r.qs[c] = ld_stream16(chunk + c * 512 + lane * 16);
        r.d = ld_stream16(chunk + 8192 + lane * 16);
    }
    __device__ static __forceinline__ void compute(const Regs &r, const ActStage &a, uint32_t *xw) {
#pragma unroll
        for (int s = 0; s < 16; s++) {
            const uint4 y = a.q[s];
#pragma unroll
            for (int w = 0; w < 4; w++)
                xw[((s >> 1) * 8 + 4 * (s & 1) + w) * 32] = (uint32_t)dp4(word_of(r.qs[s], w), word_of(y, w), 0);
        }
        xw[64 * 32] = r.d.x;
        xw[65 * 32] = r.d.y;
        xw[66 * 32] = r.d.z;
        xw[67 * 32] = r.d.w;
    }
    __device__ static __forceinline__ void chain(float &acc, const uint32_t *xg, int l, const ActView &acts, int64_t col,
                                                 int64_t group) {
        const uint16_t *dxh = acts.dh + col * (acts.k / 32) + group * 8;
#pragma unroll
        for (int blk = 0; blk < 8; blk++) {
            const uint32_t dpair = xg[(64 + (blk >> 1)) * 32];
            const float dw = f16_bits_to_f32((uint16_t)(blk & 1 ? dpair >> 16 : dpair & 0xffffu));
            const float d = __fmul_rn(dw, f16_bits_to_f32(dxh[blk]));
            acc = __fmaf_rn(d, (float)(int)xg[(blk * 8 + l) * 32], acc);
        }
    }
};

// ---------------------------------------------------------------------------
// Q4_0 and MXFP4, 8x8-gemv numerics: crates/ggml/src/repack.rs:3351-3376 and
// :1048-1068.  One chain per output: acc = fma(f32(dot32), d_w * d_x, acc) per block.
// ---------------------------------------------------------------------------
template <bool MXFP4>
struct TraitsB32 {
    static constexpr int TYPE = MXFP4 ? B200_TYPE_MXFP4 : B200_TYPE_Q4_0;
    static constexpr int CHUNK = MXFP4 ? 4352 : 4608;
    static constexpr int NW = MXFP4 ? 10 : 12;   // 8 block dots + scales (8 bytes / 8 halves)
    static constexpr int CHAINS = 1;
    static constexpr bool ACT_Q8K = false;

    struct Regs {
        uint4 qs[8], d;
    };
    __device__ static __forceinline__ void load(const uint8_t *chunk, int lane, Regs &r) {
#pragma unroll
        for (int c = 0; c < 8; c++) r.qs[c] = ld_stream16(chunk + c * 512 + lane * 16);
        if (MXFP4) {
            const uint2 e = *(const uint2 *)(chunk + 4096 + lane * 8);
            r.d = make_uint4(e.x, e.y, 0, 0);
        } else {
            r.d = ld_stream16(chunk + 4096 + lane * 16);
        }
    }
    // four 4-bit codes (one per byte of x) -> four signed bytes of 2*E2M1: crates/ggml/src/quants.rs:660
    __device__ static __forceinline__ uint32_t mxfp4_lut(uint32_t x) {
        const uint32_t lo = x & 0x07070707u;
        const uint32_t t = lo | (lo >> 4);
        const uint32_t sel = (t & 0xffu) | ((t >> 8) & 0xff00u);
        const uint32_t pos = __byte_perm(0x03020100u, 0x0c080604u, sel);
        const uint32_t neg = __byte_perm(0xfdfeff00u, 0xf4f8fafcu, sel);
        const uint32_t m = ((x & 0x08080808u) >> 3) * 0xffu;
        return (pos & ~m) | (neg & m);
    }
    __device__ static __forceinline__ void compute(const Regs &r, const ActStage &a, uint32_t *xw) {
#pragma unroll
        for (int blk = 0; blk < 8; blk++) {
            const uint4 ylo = a.q[2 * blk], yhi = a.q[2 * blk + 1];  // elements 0..15 / 16..31 of the block
            int dot = 0;
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const uint32_t q = word_of(r.qs[blk], w);
                uint32_t lo = q & 0x0f0f0f0fu, hi = (q >> 4) & 0x0f0f0f0fu;
                if (MXFP4) {
                    lo = mxfp4_lut(lo);
                    hi = mxfp4_lut(hi);
                }
                dot = dp4(lo, word_of(ylo, w), dot);
                dot = dp4(hi, word_of(yhi, w), dot);
            }
            if (!MXFP4) dot -= 8 * a.aux[8 + blk];  // (nibble - 8) * y summed = dot(nibble, y) - 8 * sum(y)
            xw[blk * 32] = (uint32_t)dot;
        }
        xw[8 * 32] = r.d.x;
        xw[9 * 32] = r.d.y;
        if (!MXFP4) {
            xw[10 * 32] = r.d.z;
            xw[11 * 32] = r.d.w;
        }
    }
    __device__ static __forceinline__ void chain(float &acc, const uint32_t *xg, int, const ActView &acts, int64_t col,
                                                 int64_t group) {
        const uint16_t *dxh = acts.dh + col * (acts.k / 32) + group * 8;
#pragma unroll
        for (int blk = 0; blk < 8; blk++) {
            float dw;
            if (MXFP4) {
                const uint32_t e4 = xg[(8 + (blk >> 2)) * 32];
                dw = e8m0_half_to_f32((e4 >> (8 * (blk & 3))) & 0xffu);
            } else {
                const uint32_t dpair = xg[(8 + (blk >> 1)) * 32];
                dw = f16_bits_to_f32((uint16_t)(blk & 1 ? dpair >> 16 : dpair & 0xffffu));
            }
            acc = __fmaf_rn((float)(int)xg[blk * 32], __fmul_rn(dw, f16_bits_to_f32(dxh[blk])), acc);
        }
    }
};

// ---------------------------------------------------------------------------
// Q6_K, tiled numerics (batch >= 8): crates/ggml/src/tiled.rs:723-839.
// Per super-block s1 = sum_sub scale * (sum u8q*y - 32*bsum) (exact int32),
// r = d_w * f32(s1), out = fma(r, d_x, out).  Same loads as the row-dot form.
// ---------------------------------------------------------------------------
struct TraitsQ6KTiled : TraitsQ6K {
    static constexpr int NW = 2;
    static constexpr int CHAINS = 1;
    __device__ static __forceinline__ void compute(const Regs &r, const ActStage &a, uint32_t *xw) {
        int s1 = 0;
#pragma unroll
        for (int n = 0; n < 2; n++)
#pragma unroll
            for (int l16 = 0; l16 < 2; l16++) {
                const uint4 A = r.ql[4 * n + l16], B = r.ql[4 * n + 2 + l16], H = r.qh[2 * n + l16];
                int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t aw = word_of(A, w), bw = word_of(B, w), hw = word_of(H, w);
                    d0 = dp4((aw & 0x0f0f0f0fu) | ((hw << 4) & 0x30303030u), word_of(a.q[8 * n + 0 + l16], w), d0);
                    d1 = dp4((bw & 0x0f0f0f0fu) | ((hw << 2) & 0x30303030u), word_of(a.q[8 * n + 2 + l16], w), d1);
                    d2 = dp4(((aw >> 4) & 0x0f0f0f0fu) | (hw & 0x30303030u), word_of(a.q[8 * n + 4 + l16], w), d2);
                    d3 = dp4(((bw >> 4) & 0x0f0f0f0fu) | ((hw >> 2) & 0x30303030u), word_of(a.q[8 * n + 6 + l16], w), d3);
                }
                // each 16-element run is one sub-block: its scale and its bsum
                s1 += scale_at(r.sc, 8 * n + 0 + l16) * (d0 - 32 * a.aux[8 * n + 0 + l16]);
                s1 += scale_at(r.sc, 8 * n + 2 + l16) * (d1 - 32 * a.aux[8 * n + 2 + l16]);
                s1 += scale_at(r.sc, 8 * n + 4 + l16) * (d2 - 32 * a.aux[8 * n + 4 + l16]);
                s1 += scale_at(r.sc, 8 * n + 6 + l16) * (d3 - 32 * a.aux[8 * n + 6 + l16]);
            }
        xw[0] = (uint32_t)s1;
        xw[32] = r.d;
    }
    __device__ static __forceinline__ void chain(float &acc, const uint32_t *xg, int, const ActView &acts, int64_t col,
                                                 int64_t group) {
        const float dx = acts.d[col * (acts.k / 256) + group];
        const float r = __fmul_rn(f16_bits_to_f32((uint16_t)xg[32]), (float)(int)xg[0]);
        acc = __fmaf_rn(r, dx, acc);
    }
};

// ---------------------------------------------------------------------------
// Q4_K, row-dot numerics (rows not a multiple of 8, fewer than 8 activation rows):
// crates/ggml/src/vec_dot.rs:872-915.  Eight scale lanes and four min lanes.
// ---------------------------------------------------------------------------
struct TraitsQ4KRowDot {
    static constexpr int TYPE = B200_TYPE_Q4_K;
    static constexpr int CHUNK = 4608;
    static constexpr int NW = 13;       // 8 lane sums, 4 min products, d|dmin
    static constexpr int CHAINS = 12;
    static constexpr bool ACT_Q8K = true;
    struct Regs {
        uint4 h, q[8];
    };
    __device__ static __forceinline__ void load(const uint8_t *chunk, int lane, Regs &r) {
        r.h = ld_stream16(chunk + lane * 16);
#pragma unroll
        for (int c = 0; c < 8; c++) r.q[c] = ld_stream16(chunk + 512 + c * 512 + lane * 16);
    }
    __device__ static __forceinline__ void compute(const Regs &r, const ActStage &a, uint32_t *xw) {
        const uint32_t u0 = r.h.y, u1 = r.h.z, u2 = r.h.w;
        const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu, mn_lo4 = u1 & 0x3f3f3f3fu;
        const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
        const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
        int sumi[8];
#pragma unroll
        for (int l = 0; l < 8; l++) sumi[l] = 0;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint32_t s4 = g < 2 ? sc_lo4 : sc_hi4;
            const int s_lo = (s4 >> (16 * (g & 1))) & 0xff, s_hi = (s4 >> (16 * (g & 1) + 8)) & 0xff;
#pragma unroll
            for (int hh = 0; hh < 2; hh++)
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t q = word_of(r.q[2 * g + hh], w);
                    const int lo = dp4(q & 0x0f0f0f0fu, word_of(a.q[4 * g + hh], w), 0);
                    const int hi = dp4((q >> 4) & 0x0f0f0f0fu, word_of(a.q[4 * g + 2 + hh], w), 0);
                    sumi[4 * hh + w] += s_lo * lo + s_hi * hi;
                }
        }
#pragma unroll
        for (int l = 0; l < 8; l++) xw[l * 32] = (uint32_t)sumi[l];
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t m4 = l < 2 ? mn_lo4 : mn_hi4;
            const int m0 = (m4 >> (16 * (l & 1))) & 0xff, m1 = (m4 >> (16 * (l & 1) + 8)) & 0xff;
            xw[(8 + l) * 32] = (uint32_t)(m0 * (a.aux[4 * l] + a.aux[4 * l + 1]) + m1 * (a.aux[4 * l + 2] + a.aux[4 * l + 3]));
        }
        xw[12 * 32] = r.h.x;
    }
    __device__ static __forceinline__ void chain(float &acc, const uint32_t *xg, int l, const ActView &acts, int64_t col,
                                                 int64_t group) {
        const float dx = acts.d[col * (acts.k / 256) + group];
        const uint32_t hd = xg[12 * 32];
        if (l < 8) {
            const float d = __fmul_rn(dx, f16_bits_to_f32((uint16_t)(hd & 0xffffu)));
            acc = __fmaf_rn(d, (float)(int)xg[l * 32], acc);
        } else {
            const float dmin = __fmul_rn(-dx, f16_bits_to_f32((uint16_t)(hd >> 16)));
            acc = __fmaf_rn(dmin, (float)(int)xg[l * 32], acc);
        }
    }
};

}  // namespace b200
