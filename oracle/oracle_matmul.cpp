// CPU oracle, part 2: row dots, the 8x8 interleaved gemv/gemm kernels, the
// tiled K-quant kernel, and the MUL_MAT / MUL_MAT_ID routing.
//
// TEST INFRASTRUCTURE ONLY (see oracle.h).  Scalar restatement of
// crates/ggml/src/vec_dot.rs, repack.rs, tiled.rs and compute.rs.
#include "oracle.h"

// vector forms of the two integer cores (oracle_simd.cpp): 1 = filled the outputs, 0 = not available / switched off
extern "C" int orc_q4kx8_ints_simd(const uint8_t *tile, const int8_t *q8, const int16_t *bs, int iacc[4][8], int imin[4][8]);
extern "C" int orc_q6k_lane_sums_simd(const uint8_t *ql, const uint8_t *qh, const int8_t *sc, const int8_t *q8, const int16_t *bsums, int sumi[8]);

#include <omp.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

static inline float f32_of(uint16_t h) { return orc_f16_to_f32(h); }
static const int8_t KVALUES_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

extern "C" int orc_num_threads() { return omp_get_max_threads(); }

// rows x k f32 -> rows of blocks, rows spread over the host threads
extern "C" int orc_quantize_rows(int type, const float *x, void *y, int64_t rows, int64_t k) {
    const size_t rs = orc_row_size(type, k);
    if (rs == 0) return -1;
    int bad = 0;
#pragma omp parallel for schedule(dynamic, 16)
    for (int64_t r = 0; r < rows; r++)
        if (orc_quantize_row(type, x + r * k, (uint8_t *)y + r * rs, k) != 0) bad = 1;
    return bad ? -1 : 0;
}

// crates/ggml/src/vec_dot.rs:564-572 hsum8 (the AVX2 horizontal-add tree)
static inline float hsum8(const float *a) {
    float r[4];
    for (int i = 0; i < 4; i++) r[i] = a[i + 4] + a[i];
    float s0 = r[0] + r[2];
    float s1 = r[1] + r[3];
    return s0 + s1;
}

// The 6-bit (scale, min) decode shared by the Q4_K kernels
// (crates/ggml/src/repack.rs:1311-1333, tiled.rs:264-288): 8 scales, 8 mins.
static inline void decode_q4k_scales(const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    for (int j = 0; j < 8; j++) {
        if (j < 4) {
            sc[j] = q[j] & 63;
            mn[j] = q[j + 4] & 63;
        } else {
            sc[j] = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
            mn[j] = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
        }
    }
}

// ===========================================================================
// row dots (AVX2 lane order specs)
// ===========================================================================

// crates/ggml/src/vec_dot.rs:595-615 vec_dot_q4_0_q8_0
static float vec_dot_q4_0_q8_0(int64_t n, const block_q4_0 *x, const block_q8_0 *y) {
    float acc[8] = {0};
    for (int64_t ib = 0; ib < n / 32; ib++) {
        float d = f32_of(x[ib].d) * f32_of(y[ib].d);
        for (int l = 0; l < 8; l++) {
            int q = 0;
            for (int i = 0; i < 4; i++) {
                int e = 4 * l + i;
                int v = e < 16 ? (x[ib].qs[e] & 0x0F) : (x[ib].qs[e - 16] >> 4);
                q += (v - 8) * (int)y[ib].qs[e];
            }
            acc[l] = fmaf(d, (float)q, acc[l]);
        }
    }
    return hsum8(acc);
}

// crates/ggml/src/vec_dot.rs:732-752 vec_dot_q8_0_q8_0
static float vec_dot_q8_0_q8_0(int64_t n, const block_q8_0 *x, const block_q8_0 *y) {
    float acc[8] = {0};
    for (int64_t ib = 0; ib < n / 32; ib++) {
        float d = f32_of(x[ib].d) * f32_of(y[ib].d);
        for (int l = 0; l < 8; l++) {
            int q = 0;
            for (int i = 0; i < 4; i++) q += (int)x[ib].qs[4 * l + i] * (int)y[ib].qs[4 * l + i];
            acc[l] = fmaf(d, (float)q, acc[l]);
        }
    }
    return hsum8(acc);
}

// crates/ggml/src/vec_dot.rs:872-915 vec_dot_q4_K_q8_K
static float vec_dot_q4_K_q8_K(int64_t n, const block_q4_K *x, const block_q8_K *y) {
    float acc[8] = {0}, acc_m[4] = {0};
    for (int64_t i = 0; i < n / QK_K; i++) {
        float d = y[i].d * f32_of(x[i].d);
        float dmin = -y[i].d * f32_of(x[i].dmin);
        uint8_t sc[8], mn[8];
        decode_q4k_scales(x[i].scales, sc, mn);
        for (int l = 0; l < 4; l++) {
            int lo = (int)y[i].bsums[4 * l] + (int)y[i].bsums[4 * l + 1];
            int hi = (int)y[i].bsums[4 * l + 2] + (int)y[i].bsums[4 * l + 3];
            int prod = (int)mn[2 * l] * lo + (int)mn[2 * l + 1] * hi;
            acc_m[l] = fmaf(dmin, (float)prod, acc_m[l]);
        }
        int sumi[8] = {0};
        for (int j = 0; j < QK_K / 64; j++) {
            int sc_lo = sc[2 * j], sc_hi = sc[2 * j + 1];
            for (int l = 0; l < 8; l++) {
                int a = 0, b = 0;
                for (int ii = 0; ii < 4; ii++) {
                    int e = 4 * l + ii;
                    a += (int)(x[i].qs[32 * j + e] & 0x0F) * (int)y[i].qs[64 * j + e];
                    b += (int)(x[i].qs[32 * j + e] >> 4) * (int)y[i].qs[64 * j + 32 + e];
                }
                sumi[l] += sc_lo * a + sc_hi * b;
            }
        }
        for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
    }
    float m0 = acc_m[0] + acc_m[2], m1 = acc_m[1] + acc_m[3];
    return hsum8(acc) + (m0 + m1);
}

// crates/ggml/src/vec_dot.rs:990-1032 vec_dot_q6_K_q8_K
static float vec_dot_q6_K_q8_K(int64_t n, const block_q6_K *x, const block_q8_K *y) {
    float acc[8] = {0};
    for (int64_t i = 0; i < n / QK_K; i++) {
        float d = y[i].d * f32_of(x[i].d);
        const uint8_t *ql = x[i].ql, *qh = x[i].qh;
        const int8_t *sc = x[i].scales;
        int sumi[8] = {0};
        if (orc_q6k_lane_sums_simd(ql, qh, sc, y[i].qs, y[i].bsums, sumi)) {   // the same exact lane sums, bias already taken off
            for (int l = 0; l < 8; l++) acc[l] = fmaf(d, (float)sumi[l], acc[l]);
            continue;
        }
        for (int j = 0; j < QK_K / 128; j++)
            for (int k = 0; k < 4; k++)
                for (int ii = 0; ii < 32; ii++) {
                    int val;
                    switch (k) {
                        case 0: val = (ql[64 * j + ii] & 0x0F) | ((qh[32 * j + ii] & 0x03) << 4); break;
                        case 1: val = (ql[64 * j + 32 + ii] & 0x0F) | (((qh[32 * j + ii] >> 2) & 0x03) << 4); break;
                        case 2: val = (ql[64 * j + ii] >> 4) | (qh[32 * j + ii] & 0x30); break;
                        default: val = (ql[64 * j + 32 + ii] >> 4) | ((qh[32 * j + ii] & 0xC0) >> 2); break;
                    }
                    int s = sc[8 * j + 2 * k + (ii >= 16 ? 1 : 0)];
                    sumi[ii / 4] += s * (int)y[i].qs[128 * j + 32 * k + ii] * val;
                }
        for (int l = 0; l < 8; l++) {
            int sub = ((int)y[i].bsums[2 * l] * (int)sc[2 * l] + (int)y[i].bsums[2 * l + 1] * (int)sc[2 * l + 1]) << 5;
            sumi[l] -= sub;
            acc[l] = fmaf(d, (float)sumi[l], acc[l]);
        }
    }
    return hsum8(acc);
}

// crates/ggml/src/compute.rs:7123-7147 vec_dot_mxfp4_q8_0 (scalar generic:
// sumf += d * sumi, not fused)
static float vec_dot_mxfp4_q8_0(int64_t n, const block_mxfp4 *x, const block_q8_0 *y) {
    float sumf = 0.0f;
    for (int64_t ib = 0; ib < n / 32; ib++) {
        float d = f32_of(y[ib].d) * orc_e8m0_to_f32_half(x[ib].e);
        int s1 = 0, s2 = 0;
        for (int j = 0; j < 16; j++) {
            s1 += (int)y[ib].qs[j] * (int)KVALUES_MXFP4[x[ib].qs[j] & 0xF];
            s2 += (int)y[ib].qs[j + 16] * (int)KVALUES_MXFP4[x[ib].qs[j] >> 4];
        }
        sumf += d * (float)(s1 + s2);
    }
    return sumf;
}

extern "C" float orc_vec_dot(int type, int64_t k, const void *w, const void *a) {
    switch (type) {
        case ORC_Q4_0: return vec_dot_q4_0_q8_0(k, (const block_q4_0 *)w, (const block_q8_0 *)a);
        case ORC_Q8_0: return vec_dot_q8_0_q8_0(k, (const block_q8_0 *)w, (const block_q8_0 *)a);
        case ORC_Q4_K: return vec_dot_q4_K_q8_K(k, (const block_q4_K *)w, (const block_q8_K *)a);
        case ORC_Q6_K: return vec_dot_q6_K_q8_K(k, (const block_q6_K *)w, (const block_q8_K *)a);
        case ORC_MXFP4: return vec_dot_mxfp4_q8_0(k, (const block_mxfp4 *)w, (const block_q8_0 *)a);
        default: return NAN;
    }
}

// ===========================================================================
// 8x8 kernels on the interleaved layouts
// ===========================================================================

// Decode one 12-byte group of block_q4_Kx8.scales into the 8 columns'
// (scale, min) — crates/ggml/src/repack.rs:1311-1333,1612-1622.
static inline void q4kx8_scales(const uint8_t *tile, int sb, uint8_t *s, uint8_t *m) {
    const int off = sb < 4 ? 12 * sb : 12 * (sb - 4) + 48;
    uint32_t u[4];
    std::memcpy(u, tile + 32 + off, 12);
    const uint32_t K1 = 0x3f3f3f3f, K2 = 0x0f0f0f0f, K3 = 0x03030303;
    u[3] = ((u[2] >> 4) & K2) | (((u[1] >> 6) & K3) << 4);
    uint32_t aux = u[1] & K1;
    u[1] = (u[2] & K2) | (((u[0] >> 6) & K3) << 4);
    u[2] = aux;
    u[0] &= K1;
    std::memcpy(s, &u[0], 8);
    std::memcpy(m, &u[2], 8);
}

// Integer part of one (tile, activation super-block): iacc/imin per sub-block
// pair g for the 8 columns.  q8 = 256 plain-order quants, bs = 16 bsums.
static inline void q4kx8_ints(const uint8_t *tile, const int8_t *q8, const int16_t *bs,
                              int iacc[4][8], int imin[4][8]) {
    // the same exact integers from the vector form when the host has one (oracle_simd.cpp; orc_set_simd(0) turns it off)
    if (orc_q4kx8_ints_simd(tile, q8, bs, iacc, imin)) return;
    for (int g = 0; g < 4; g++) {
        uint8_t s_lo[8], m_lo[8], s_hi[8], m_hi[8];
        q4kx8_scales(tile, 2 * g, s_lo, m_lo);
        q4kx8_scales(tile, 2 * g + 1, s_hi, m_hi);
        int d_lo[8] = {0}, d_hi[8] = {0};
        const uint8_t *qs = tile + 128 + 256 * g;
        for (int c = 0; c < 8; c++) {
            int lo = 0, hi = 0;
            for (int m = 0; m < 32; m++) {
                uint8_t byte = qs[8 * c + 64 * (m / 8) + (m % 8)];
                lo += (int)(byte & 0xF) * (int)q8[64 * g + m];
                hi += (int)(byte >> 4) * (int)q8[64 * g + 32 + m];
            }
            d_lo[c] = lo;
            d_hi[c] = hi;
        }
        int b_lo = (int)bs[4 * g] + (int)bs[4 * g + 1];
        int b_hi = (int)bs[4 * g + 2] + (int)bs[4 * g + 3];
        for (int c = 0; c < 8; c++) {
            iacc[g][c] = d_lo[c] * (int)s_lo[c] + d_hi[c] * (int)s_hi[c];
            imin[g][c] = (int)m_lo[c] * b_lo + (int)m_hi[c] * b_hi;
        }
    }
}

// crates/ggml/src/repack.rs:1638-1688 gemv_q4_K_8x8_q8_K: one fma per
// super-block for the scale term and one for the min term.
static void gemv_q4_K_8x8_q8_K(int64_t n, float *s, const uint8_t *vx, const uint8_t *vy, int64_t nc) {
    const int64_t nb = n / QK_K;
    for (int64_t x = 0; x < nc / 8; x++) {
        const uint8_t *bmat = vx + x * nb * 1152;
        float sumf[8] = {0}, summin[8] = {0};
        for (int64_t b = 0; b < nb; b++) {
            const uint8_t *tile = bmat + b * 1152;
            const block_q8_K *q8 = (const block_q8_K *)(vy + b * 292);
            int ia[4][8], im[4][8];
            q4kx8_ints(tile, q8->qs, q8->bsums, ia, im);
            for (int c = 0; c < 8; c++) {
                int iacc = ia[0][c] + ia[1][c] + ia[2][c] + ia[3][c];
                int imin = im[0][c] + im[1][c] + im[2][c] + im[3][c];
                uint16_t dh, mh;
                std::memcpy(&dh, tile + 2 * c, 2);
                std::memcpy(&mh, tile + 16 + 2 * c, 2);
                sumf[c] = fmaf((float)iacc, f32_of(dh) * q8->d, sumf[c]);
                summin[c] = fmaf((float)imin, f32_of(mh) * q8->d, summin[c]);
            }
        }
        for (int c = 0; c < 8; c++) s[x * 8 + c] = sumf[c] - summin[c];
    }
}

// crates/ggml/src/repack.rs:1692-1768 gemm_q4_K_8x8_q8_K: one fma per
// (super-block, sub-block pair); activations are block_q8_Kx4 tiles.
static void gemm_q4_K_8x8_q8_K(int64_t n, float *s, int64_t bs, const uint8_t *vx, const uint8_t *vy,
                               int64_t nr, int64_t nc) {
    const int64_t nb = n / QK_K;
    // the 4 rows of an activation tile in plain order, once per tile: element el of row r is at
    // qs[(el/8)*32 + r*8 + el%8], its 16-element sums at 16*(el/64) + 4r + (el/16)%4
    std::vector<int8_t> q8(nb * 4 * 256);
    std::vector<int16_t> bsr(nb * 4 * 16);
    for (int64_t y = 0; y < nr / 4; y++) {
        const uint8_t *ablk = vy + y * nb * 1168;
        for (int64_t b = 0; b < nb; b++) {
            const int8_t *aq = (const int8_t *)(ablk + b * 1168 + 16);
            const int16_t *abs_ = (const int16_t *)(ablk + b * 1168 + 1040);
            for (int r = 0; r < 4; r++) {
                int8_t *q = q8.data() + (b * 4 + r) * 256;
                for (int p = 0; p < 32; p++) std::memcpy(q + 8 * p, aq + p * 32 + r * 8, 8);
                for (int j = 0; j < 16; j++) bsr[(b * 4 + r) * 16 + j] = abs_[16 * (j / 4) + 4 * r + j % 4];
            }
        }
        for (int64_t x = 0; x < nc / 8; x++) {
            const uint8_t *bmat = vx + x * nb * 1152;
            float acc[4][8] = {{0}}, accmin[4][8] = {{0}};
            for (int64_t b = 0; b < nb; b++) {
                const uint8_t *tile = bmat + b * 1152;
                const float *ad = (const float *)(ablk + b * 1168);
                float dcol[8], mcol[8];
                for (int c = 0; c < 8; c++) {
                    uint16_t dh, mh;
                    std::memcpy(&dh, tile + 2 * c, 2);
                    std::memcpy(&mh, tile + 16 + 2 * c, 2);
                    dcol[c] = f32_of(dh);
                    mcol[c] = f32_of(mh);
                }
                for (int r = 0; r < 4; r++) {
                    int ia[4][8], im[4][8];
                    q4kx8_ints(tile, q8.data() + (b * 4 + r) * 256, bsr.data() + (b * 4 + r) * 16, ia, im);
                    for (int g = 0; g < 4; g++)
                        for (int c = 0; c < 8; c++) {
                            acc[r][c] = fmaf((float)ia[g][c], dcol[c] * ad[r], acc[r][c]);
                            accmin[r][c] = fmaf((float)im[g][c], mcol[c] * ad[r], accmin[r][c]);
                        }
                }
            }
            for (int r = 0; r < 4; r++)
                for (int c = 0; c < 8; c++) s[(y * 4 + r) * bs + x * 8 + c] = acc[r][c] - accmin[r][c];
        }
    }
}

// One 32-element block of an 8-row Q4_0/MXFP4 tile against one activation
// block: crates/ggml/src/repack.rs:1048-1068 (MXFP4), :3351-3376 (Q4_0).
// The tile keeps, after its 8 headers, rows 0..7 of nibble bytes 0..7 and
// then rows 0..7 of nibble bytes 8..15.
static inline void accum_block_b32x8(int type, const uint8_t *tile, float d_act, const int8_t *aq, float *acc) {
    const int hdr = type == ORC_Q4_0 ? 2 : 1;
    const uint8_t *qs = tile + 8 * hdr;
    for (int c = 0; c < 8; c++) {
        int dot = 0;
        for (int e = 0; e < 32; e++) {
            int j = e % 16;
            uint8_t byte = qs[(j / 8) * 64 + c * 8 + j % 8];
            int nib = e < 16 ? (byte & 0xF) : (byte >> 4);
            int v = type == ORC_Q4_0 ? (nib < 8 ? nib : nib - 16) : KVALUES_MXFP4[nib];
            dot += v * (int)aq[e];
        }
        float dcol;
        if (type == ORC_Q4_0) {
            uint16_t dh;
            std::memcpy(&dh, tile + 2 * c, 2);
            dcol = f32_of(dh);
        } else {
            dcol = orc_e8m0_to_f32_half(tile[c]);
        }
        acc[c] = fmaf((float)dot, dcol * d_act, acc[c]);
    }
}

static void gemv_b32_8x8_q8_0(int type, int64_t n, float *s, const uint8_t *vx, const uint8_t *vy, int64_t nc) {
    const int64_t nb = n / 32;
    const int tile = type == ORC_Q4_0 ? 144 : 136;
    const block_q8_0 *a = (const block_q8_0 *)vy;
    for (int64_t x = 0; x < nc / 8; x++) {
        float acc[8] = {0};
        for (int64_t b = 0; b < nb; b++)
            accum_block_b32x8(type, vx + (x * nb + b) * tile, f32_of(a[b].d), a[b].qs, acc);
        std::memcpy(s + x * 8, acc, 32);
    }
}

// crates/ggml/src/repack.rs:1136-1184 (MXFP4) / :3380-3421 (Q4_0) gemm: same
// per-element arithmetic as the gemv, activations in block_q8_0x4 tiles.
static void gemm_b32_8x8_q8_0(int type, int64_t n, float *s, int64_t bs, const uint8_t *vx, const uint8_t *vy,
                              int64_t nr, int64_t nc) {
    const int64_t nb = n / 32;
    const int tile = type == ORC_Q4_0 ? 144 : 136;
    for (int64_t y = 0; y < nr / 4; y++)
        for (int64_t x = 0; x < nc / 8; x++) {
            float acc[4][8] = {{0}};
            for (int64_t b = 0; b < nb; b++) {
                const uint8_t *a = vy + (y * nb + b) * 136;
                for (int r = 0; r < 4; r++) {
                    uint16_t dh;
                    std::memcpy(&dh, a + 2 * r, 2);
                    int8_t q[32];
                    for (int e = 0; e < 32; e++) q[e] = (int8_t)a[8 + (e / 8) * 32 + r * 8 + e % 8];
                    accum_block_b32x8(type, vx + (x * nb + b) * tile, f32_of(dh), q, acc[r]);
                }
            }
            for (int r = 0; r < 4; r++) std::memcpy(s + (y * 4 + r) * bs + x * 8, acc[r], 32);
        }
}

extern "C" int orc_gemv_8x8(int type, int64_t k, float *s, const void *vx, const void *vy, int64_t nc) {
    if (nc % 8) return -1;
    if (type == ORC_Q4_K) { gemv_q4_K_8x8_q8_K(k, s, (const uint8_t *)vx, (const uint8_t *)vy, nc); return 0; }
    if (type == ORC_Q4_0 || type == ORC_MXFP4) { gemv_b32_8x8_q8_0(type, k, s, (const uint8_t *)vx, (const uint8_t *)vy, nc); return 0; }
    return -1;
}
extern "C" int orc_gemm_8x8(int type, int64_t k, float *s, int64_t bs, const void *vx, const void *vy,
                            int64_t nr, int64_t nc) {
    if (nc % 8 || nr % 4) return -1;
    if (type == ORC_Q4_K) { gemm_q4_K_8x8_q8_K(k, s, bs, (const uint8_t *)vx, (const uint8_t *)vy, nr, nc); return 0; }
    if (type == ORC_Q4_0 || type == ORC_MXFP4) { gemm_b32_8x8_q8_0(type, k, s, bs, (const uint8_t *)vx, (const uint8_t *)vy, nr, nc); return 0; }
    return -1;
}

// ===========================================================================
// tiled K-quant kernel, per output element
// crates/ggml/src/tiled.rs:723-839 (micro kernel) driven in ascending K by
// :1656-1780; activations are plain Q8_K rows.  Per super-block:
//   s1 = sum_sub scale * (sum u8q*y - BIAS*bsum)   (exact int32)
//   s2 = sum_sub min * bsum                        (Q4_K only)
//   r = d_w * f32(s1); r = fma(-dmin_w, f32(s2), r); out = fma(r, d_x, out)
// ===========================================================================
static float tiled_dot_q4_K(int64_t n, const block_q4_K *x, const block_q8_K *y) {
    float out = 0.0f;
    for (int64_t i = 0; i < n / QK_K; i++) {
        uint8_t sc[8], mn[8];
        decode_q4k_scales(x[i].scales, sc, mn);
        int s1 = 0, s2 = 0;
        for (int sb = 0; sb < 8; sb++) {
            int raw = 0;
            const uint8_t *q = x[i].qs + 32 * (sb / 2);
            for (int l = 0; l < 32; l++) {
                int v = (sb & 1) ? (q[l] >> 4) : (q[l] & 0xF);
                raw += v * (int)y[i].qs[32 * sb + l];
            }
            s1 += raw * (int)sc[sb];
            s2 += ((int)y[i].bsums[2 * sb] + (int)y[i].bsums[2 * sb + 1]) * (int)mn[sb];
        }
        float r = f32_of(x[i].d) * (float)s1;
        r = fmaf(-f32_of(x[i].dmin), (float)s2, r);
        out = fmaf(r, y[i].d, out);
    }
    return out;
}

static float tiled_dot_q6_K(int64_t n, const block_q6_K *x, const block_q8_K *y) {
    float out = 0.0f;
    for (int64_t i = 0; i < n / QK_K; i++) {
        const uint8_t *ql = x[i].ql, *qh = x[i].qh;
        int s1 = 0;
        int lanes[8];
        // the vector row-dot core yields the same exact total, split over eight lanes
        if (orc_q6k_lane_sums_simd(ql, qh, x[i].scales, y[i].qs, y[i].bsums, lanes)) {
            for (int l = 0; l < 8; l++) s1 += lanes[l];
            out = fmaf(f32_of(x[i].d) * (float)s1, y[i].d, out);
            continue;
        }
        for (int sb = 0; sb < 16; sb++) {
            int raw = 0;
            for (int t = 0; t < 16; t++) {
                int el = 16 * sb + t;
                int j = el / 128, r = el % 128, k = r / 32, ii = r % 32;
                int val;
                switch (k) {
                    case 0: val = (ql[64 * j + ii] & 0x0F) | ((qh[32 * j + ii] & 0x03) << 4); break;
                    case 1: val = (ql[64 * j + 32 + ii] & 0x0F) | (((qh[32 * j + ii] >> 2) & 0x03) << 4); break;
                    case 2: val = (ql[64 * j + ii] >> 4) | (qh[32 * j + ii] & 0x30); break;
                    default: val = (ql[64 * j + 32 + ii] >> 4) | ((qh[32 * j + ii] & 0xC0) >> 2); break;
                }
                raw += val * (int)y[i].qs[el];
            }
            raw -= 32 * (int)y[i].bsums[sb];
            s1 += raw * (int)x[i].scales[sb];
        }
        float r = f32_of(x[i].d) * (float)s1;
        out = fmaf(r, y[i].d, out);
    }
    return out;
}

// ===========================================================================
// MUL_MAT routing — crates/ggml/src/compute.rs:1420-1841
// ===========================================================================
static int pick_route(int type, int64_t N, int64_t M) {
    switch (type) {
        case ORC_Q4_K:
            if (N % 8 == 0) return ORC_ROUTE_REPACK;      // compute.rs:5093-5131
            return M >= 8 ? ORC_ROUTE_TILED : ORC_ROUTE_ROWDOT;
        case ORC_Q6_K: return M >= 8 ? ORC_ROUTE_TILED : ORC_ROUTE_ROWDOT;  // compute.rs:1596
        case ORC_Q8_0: return ORC_ROUTE_ROWDOT;  // tinyBLAS values == row dot (tinyblas.rs:64-74)
        case ORC_Q4_0:
        case ORC_MXFP4: return N % 8 == 0 ? ORC_ROUTE_REPACK : ORC_ROUTE_ROWDOT;
        default: return -1;
    }
}

extern "C" int orc_pick_route(int type, int64_t N, int64_t M) { return pick_route(type, N, M); }

static inline bool is_kquant(int type) { return type == ORC_Q4_K || type == ORC_Q6_K; }

// Quantize M activation rows the plain way for `type` (A2 for K-quants, A1 else).
static void quantize_acts_plain(int type, const float *X, int64_t K, int64_t M, std::vector<uint8_t> &wd, size_t &rs) {
    rs = is_kquant(type) ? (size_t)(K / 256) * 292 : (size_t)(K / 32) * 34;
    wd.resize(rs * M);
#pragma omp parallel for schedule(static)
    for (int64_t m = 0; m < M; m++) {
        if (is_kquant(type)) orc_quantize_row_q8_K(X + m * K, wd.data() + m * rs, K);
        else orc_quantize_row_q8_0(X + m * K, wd.data() + m * rs, K);
    }
}

// Weights already in the 8x8 layout.  Q4_K: compute.rs:5322-5447; Q4_0:
// compute.rs:5192-5320; MXFP4: compute.rs:1767-1803 (gemv per activation row).
static void mul_mat_repacked(int type, int64_t N, int64_t K, int64_t M, const uint8_t *rep, const float *X,
                             float *out) {
    const int64_t nr4 = (type == ORC_MXFP4) ? 0 : M - M % 4;
    std::vector<uint8_t> wd4, wdp;
    size_t rs = 0;
    if (nr4 > 0) {
        if (type == ORC_Q4_K) {
            wd4.resize((size_t)(nr4 / 4) * (K / 256) * 1168);
#pragma omp parallel for schedule(static)
            for (int64_t g = 0; g < nr4 / 4; g++)
                orc_quantize_mat_q8_K_4x8(X + g * 4 * K, K, 4, wd4.data() + (size_t)g * (K / 256) * 1168);
        } else {
            wd4.resize((size_t)(nr4 / 4) * (K / 32) * 136);
#pragma omp parallel for schedule(static)
            for (int64_t g = 0; g < nr4 / 4; g++)
                orc_quantize_mat_q8_0_4x8(X + g * 4 * K, K, 4, wd4.data() + (size_t)g * (K / 32) * 136);
        }
    }
    if (M > nr4) quantize_acts_plain(type, X + nr4 * K, K, M - nr4, wdp, rs);
    const size_t group_bytes = (size_t)8 * orc_row_size(type, K);
    // 8-row weight groups are independent (compute.rs:5404-5440 chunks them 8-aligned)
    const int64_t groups = N / 8;
    const int64_t chunk = std::max<int64_t>(1, groups / (4 * (int64_t)omp_get_max_threads()));
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t c0 = 0; c0 < groups; c0 += chunk) {
        const int64_t c1 = std::min(groups, c0 + chunk);
        const uint8_t *bmat = rep + c0 * group_bytes;
        const int64_t ncols = (c1 - c0) * 8;
        if (nr4 > 0) {
            if (type == ORC_Q4_K) gemm_q4_K_8x8_q8_K(K, out + c0 * 8, N, bmat, wd4.data(), nr4, ncols);
            else gemm_b32_8x8_q8_0(type, K, out + c0 * 8, N, bmat, wd4.data(), nr4, ncols);
        }
        for (int64_t r = nr4; r < M; r++) {
            const uint8_t *a = wdp.data() + (r - nr4) * rs;
            if (type == ORC_Q4_K) gemv_q4_K_8x8_q8_K(K, out + r * N + c0 * 8, bmat, a, ncols);
            else gemv_b32_8x8_q8_0(type, K, out + r * N + c0 * 8, bmat, a, ncols);
        }
    }
}

extern "C" int orc_mul_mat_repacked(int type, int64_t N, int64_t K, int64_t M, const void *Wrep, const float *X,
                                    float *out, int n_threads) {
    if (pick_route(type, N, M) != ORC_ROUTE_REPACK) return -1;
    if (n_threads > 0) omp_set_num_threads(n_threads);
    mul_mat_repacked(type, N, K, M, (const uint8_t *)Wrep, X, out);
    return ORC_ROUTE_REPACK;
}

extern "C" int orc_mul_mat(int type, int64_t N, int64_t K, int64_t M, const void *W, const float *X, float *out,
                           int route, int n_threads) {
    const int be = orc_block_elems(type);
    if (be == 0 || K % be != 0) return -1;
    if (route == ORC_ROUTE_AUTO) route = pick_route(type, N, M);
    if (route < 0) return -1;
    if (n_threads > 0) omp_set_num_threads(n_threads);
    const size_t wrs = orc_row_size(type, K);
    if (route == ORC_ROUTE_REPACK) {
        if (N % 8 != 0 || !(type == ORC_Q4_K || type == ORC_Q4_0 || type == ORC_MXFP4)) return -1;
        std::vector<uint8_t> rep((size_t)N * wrs);
        if (orc_repack_8x8(type, W, N, K, rep.data()) != 0) return -1;
        mul_mat_repacked(type, N, K, M, rep.data(), X, out);
        return route;
    }
    if (route == ORC_ROUTE_TILED && !is_kquant(type)) return -1;
    std::vector<uint8_t> wd;
    size_t rs;
    quantize_acts_plain(type, X, K, M, wd, rs);
    const uint8_t *Wb = (const uint8_t *)W;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        const void *wrow = Wb + n * wrs;
        for (int64_t m = 0; m < M; m++) {
            const void *arow = wd.data() + m * rs;
            float v;
            if (route == ORC_ROUTE_TILED) {
                v = type == ORC_Q4_K ? tiled_dot_q4_K(K, (const block_q4_K *)wrow, (const block_q8_K *)arow)
                                     : tiled_dot_q6_K(K, (const block_q6_K *)wrow, (const block_q8_K *)arow);
            } else {
                v = orc_vec_dot(type, K, wrow, arow);
            }
            out[m * N + n] = v;
        }
    }
    return route;
}

// ===========================================================================
// MUL_MAT_ID — crates/ggml/src/compute.rs:1917-2202
// Every b row is quantized once; for (slot i1, token i2): expert = ids[i2][i1],
// activation row i11 = i1 % ne11 of token i2, output out[i2][i1][:].
// MXFP4 / Q4_0 / Q4_K experts with N % 8 == 0 run the 8x8 gemv per pair
// (:2131-2181); K-quant experts with >= 8 routed rows take the tiled kernel
// (:2036-2104); everything else is the row dot (:2183-2190).
// ===========================================================================
extern "C" int orc_mul_mat_id(int type, int64_t N, int64_t K, int64_t n_expert, int64_t ne11, int64_t n_tok,
                              int64_t n_ids, const void *W, const float *B, const int32_t *ids, float *out,
                              int route, int n_threads) {
    const int be = orc_block_elems(type);
    if (be == 0 || K % be != 0) return -1;
    if (n_threads > 0) omp_set_num_threads(n_threads);
    const size_t wrs = orc_row_size(type, K);
    const uint8_t *Wb = (const uint8_t *)W;
    std::vector<uint8_t> wd;
    size_t rs;
    quantize_acts_plain(type, B, K, ne11 * n_tok, wd, rs);

    std::vector<int64_t> cnt(n_expert, 0);
    for (int64_t t = 0; t < n_tok; t++)
        for (int64_t s = 0; s < n_ids; s++) {
            int32_t e = ids[t * n_ids + s];
            if (e < 0 || e >= n_expert) return -1;
            cnt[e]++;
        }
    const bool repackable = (type == ORC_MXFP4 || type == ORC_Q4_0 || type == ORC_Q4_K) && N % 8 == 0;
    if (route == ORC_ROUTE_AUTO)
        route = repackable ? ORC_ROUTE_REPACK : (is_kquant(type) ? ORC_ROUTE_TILED : ORC_ROUTE_ROWDOT);
    std::vector<uint8_t> rep;
    if (route == ORC_ROUTE_REPACK) {
        if (!repackable) return -1;
        rep.resize((size_t)n_expert * N * wrs);
        for (int64_t e = 0; e < n_expert; e++)
            orc_repack_8x8(type, Wb + e * N * wrs, N, K, rep.data() + e * N * wrs);
    }
#pragma omp parallel for schedule(dynamic, 4) collapse(2)
    for (int64_t t = 0; t < n_tok; t++)
        for (int64_t s = 0; s < n_ids; s++) {
            const int32_t e = ids[t * n_ids + s];
            const int64_t i11 = s % ne11;
            const uint8_t *arow = wd.data() + (t * ne11 + i11) * rs;
            float *o = out + (t * n_ids + s) * N;
            if (route == ORC_ROUTE_REPACK) {
                if (type == ORC_Q4_K) gemv_q4_K_8x8_q8_K(K, o, rep.data() + (size_t)e * N * wrs, arow, N);
                else gemv_b32_8x8_q8_0(type, K, o, rep.data() + (size_t)e * N * wrs, arow, N);
                continue;
            }
            // tiled per expert only when that expert has >= 8 routed rows
            const bool tiled = route == ORC_ROUTE_TILED && is_kquant(type) && cnt[e] >= 8;
            for (int64_t n = 0; n < N; n++) {
                const void *wrow = Wb + ((size_t)e * N + n) * wrs;
                if (tiled) {
                    o[n] = type == ORC_Q4_K ? tiled_dot_q4_K(K, (const block_q4_K *)wrow, (const block_q8_K *)arow)
                                            : tiled_dot_q6_K(K, (const block_q6_K *)wrow, (const block_q8_K *)arow);
                } else {
                    o[n] = orc_vec_dot(type, K, wrow, arow);
                }
            }
        }
    return route;
}
