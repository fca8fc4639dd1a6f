// CPU oracle, part 1: block formats, weight quantizers, dequantizers, the four
// activation quantizers and the 8x8 interleaved layouts.
//
// TEST INFRASTRUCTURE ONLY (see oracle.h).  Scalar restatement of
// crates/ggml/src/quants.rs, quants_k.rs and repack.rs of the reference.
#include "oracle.h"

#include <immintrin.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

// ---------------------------------------------------------------------------
// f16 <-> f32: IEEE round-to-nearest-even, what the `half` crate (2.7.1) does
// for f16::from_f32 / to_f32 (crates/ggml/src/quants.rs:21-27).  F16C is exact.
// ---------------------------------------------------------------------------
extern "C" uint16_t orc_f32_to_f16(float x) {
    return (uint16_t)_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
}
extern "C" float orc_f16_to_f32(uint16_t h) { return _cvtsh_ss(h); }

static inline uint16_t fp16(float x) { return orc_f32_to_f16(x); }
static inline float f32_of(uint16_t h) { return orc_f16_to_f32(h); }

// crates/ggml/src/quants.rs:13-18 nearest_int (magic-number RNE, |f| < 2^22)
static inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    int32_t i;
    std::memcpy(&i, &val, 4);
    return (i & 0x007fffff) - 0x00400000;
}

// crates/ggml/src/quants.rs:682-691 e8m0_to_fp32_half: 2^(e-128)
extern "C" float orc_e8m0_to_f32_half(uint8_t x) {
    uint32_t bits = x < 2 ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// crates/ggml/src/quants.rs:660
static const int8_t KVALUES_MXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

extern "C" int orc_block_elems(int type) {
    switch (type) {
        case ORC_F32: case ORC_F16: return 1;
        case ORC_Q4_0: case ORC_Q8_0: case ORC_MXFP4: return 32;
        case ORC_Q4_K: case ORC_Q6_K: case ORC_Q8_K: return 256;
        default: return 0;
    }
}
static size_t block_bytes(int type) {
    switch (type) {
        case ORC_F32: return 4;
        case ORC_F16: return 2;
        case ORC_Q4_0: return 18;
        case ORC_Q8_0: return 34;
        case ORC_MXFP4: return 17;
        case ORC_Q4_K: return 144;
        case ORC_Q6_K: return 210;
        case ORC_Q8_K: return 292;
        default: return 0;
    }
}
// crates/ggml/src/types.rs:172 row_size
extern "C" size_t orc_row_size(int type, int64_t k) {
    int be = orc_block_elems(type);
    if (be == 0) return 0;
    return (size_t)(k / be) * block_bytes(type);
}

// ===========================================================================
// weight quantizers
// ===========================================================================

// crates/ggml/src/quants.rs:124-152 quantize_row_q4_0_ref
static void quantize_row_q4_0_ref(const float *x, block_q4_0 *y, int64_t k) {
    const int qk = QK4_0;
    for (int64_t i = 0; i < k / qk; i++) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < qk; j++) {
            float v = x[i * qk + j];
            if (amax < std::fabs(v)) { amax = std::fabs(v); max = v; }
        }
        const float d = max / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < qk / 2; j++) {
            const float x0 = x[i * qk + j] * id;
            const float x1 = x[i * qk + qk / 2 + j] * id;
            // Rust `as i8` saturates; the value range here is [0.5, 16.5]
            int xi0 = (int)std::max(-128.0f, std::min(127.0f, std::trunc(x0 + 8.5f)));
            int xi1 = (int)std::max(-128.0f, std::min(127.0f, std::trunc(x1 + 8.5f)));
            uint8_t b0 = (uint8_t)std::min(xi0, 15) & 0x0F;
            uint8_t b1 = (uint8_t)std::min(xi1, 15) & 0x0F;
            y[i].qs[j] = b0 | (b1 << 4);
        }
        y[i].d = fp16(d);
    }
}

// crates/ggml/src/quants.rs:309-326 quantize_row_q8_0_ref (file-format
// quantizer: id = 1/d, round half away from zero)
static void quantize_row_q8_0_ref(const float *x, block_q8_0 *y, int64_t k) {
    for (int64_t i = 0; i < k / QK8_0; i++) {
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; j++) amax = std::max(amax, std::fabs(x[i * QK8_0 + j]));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        for (int j = 0; j < QK8_0; j++) {
            float r = std::round(x[i * QK8_0 + j] * id);
            y[i].qs[j] = (int8_t)std::max(-128.0f, std::min(127.0f, r));
        }
        y[i].d = fp16(d);
    }
}

// crates/ggml/src/quants_k.rs:1396-1487 make_qkx2_quants
static float make_qkx2_quants(int n, int nmax, const float *x, const float *weights, uint8_t *L,
                              float *the_min, uint8_t *Laux, float rmin, float rdelta, int nstep,
                              bool use_mad) {
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        float w = weights[i];
        sum_w += w;
        sum_x += w * x[i];
    }
    if (min > 0.0f) min = 0.0f;
    if (max == min) {
        for (int i = 0; i < n; i++) L[i] = 0;
        *the_min = -min;
        return 0.0f;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = nearest_int(iscale * (x[i] - min));
        L[i] = (uint8_t)std::max(0, std::min(nmax, l));
        float diff = scale * (float)L[i] + min - x[i];
        diff = use_mad ? std::fabs(diff) : diff * diff;
        best_error += weights[i] * diff;
    }
    if (nstep < 1) { *the_min = -min; return scale; }
    for (int is = 0; is <= nstep; is++) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max - min);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int l = std::max(0, std::min(nmax, nearest_int(iscale * (x[i] - min))));
            Laux[i] = (uint8_t)l;
            float w = weights[i];
            sum_l += w * (float)l;
            sum_l2 += w * (float)l * (float)l;
            sum_xl += w * (float)l * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0.0f) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0.0f) { this_min = 0.0f; this_scale = sum_xl / sum_l2; }
            float cur_error = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                diff = use_mad ? std::fabs(diff) : diff * diff;
                cur_error += weights[i] * diff;
            }
            if (cur_error < best_error) {
                std::memcpy(L, Laux, n);
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

// crates/ggml/src/quants.rs:421-429 get_scale_min_k4
static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

// crates/ggml/src/quants_k.rs:1861-1949 quantize_row_q4_K_ref
static void quantize_row_q4_K_ref(const float *x, block_q4_K *y, int64_t k) {
    uint8_t L[QK_K], Laux[32];
    float weights[32], mins[QK_K / 32], scales[QK_K / 32];
    for (int64_t i = 0; i < k / QK_K; i++) {
        const float *xb = x + i * QK_K;
        float max_scale = 0.0f, max_min = 0.0f;
        for (int j = 0; j < QK_K / 32; j++) {
            float sum_x2 = 0.0f;
            for (int l = 0; l < 32; l++) sum_x2 += xb[32 * j + l] * xb[32 * j + l];
            float av_x = std::sqrt(sum_x2 / 32.0f);
            for (int l = 0; l < 32; l++) weights[l] = av_x + std::fabs(xb[32 * j + l]);
            scales[j] = make_qkx2_quants(32, 15, xb + 32 * j, weights, L + 32 * j, &mins[j], Laux,
                                         -1.0f, 0.1f, 20, false);
            if (scales[j] > max_scale) max_scale = scales[j];
            if (mins[j] > max_min) max_min = mins[j];
        }
        float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
        float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
        uint8_t sb[K_SCALE_SIZE] = {0};
        for (int j = 0; j < QK_K / 32; j++) {
            uint8_t ls = (uint8_t)nearest_int(inv_scale * scales[j]);
            uint8_t lm = (uint8_t)nearest_int(inv_min * mins[j]);
            ls = std::min<uint8_t>(ls, 63);
            lm = std::min<uint8_t>(lm, 63);
            if (j < 4) {
                sb[j] = ls;
                sb[j + 4] = lm;
            } else {
                sb[j + 4] = (ls & 0xF) | ((lm & 0xF) << 4);
                sb[j - 4] |= (ls >> 4) << 6;
                sb[j] |= (lm >> 4) << 6;
            }
        }
        uint16_t dh = fp16(max_scale / 63.0f);
        uint16_t dminh = fp16(max_min / 63.0f);
        for (int j = 0; j < QK_K / 32; j++) {
            uint8_t sc, m;
            get_scale_min_k4(j, sb, &sc, &m);
            float d = f32_of(dh) * (float)sc;
            if (d == 0.0f) continue;
            float dm = f32_of(dminh) * (float)m;
            for (int ii = 0; ii < 32; ii++) {
                int l = nearest_int((xb[32 * j + ii] + dm) / d);
                L[32 * j + ii] = (uint8_t)std::max(0, std::min(15, l));
            }
        }
        uint8_t *q = y[i].qs;
        for (int j = 0; j < QK_K; j += 64) {
            for (int l = 0; l < 32; l++) q[l] = L[j + l] | (L[j + l + 32] << 4);
            q += 32;
        }
        y[i].d = dh;
        y[i].dmin = dminh;
        std::memcpy(y[i].scales, sb, K_SCALE_SIZE);
    }
}

static const float GROUP_MAX_EPS = 1e-15f;  // crates/ggml/src/quants_k.rs:25

// crates/ggml/src/quants_k.rs:1170-1260 make_qx_quants with qw == None
static float make_qx_quants(int n, int nmax, const float *x, int8_t *L, int rmse_type) {
    float max = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; i++) {
        float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; i++) L[i] = 0;
        return 0.0f;
    }
    float iscale = -(float)nmax / max;
    if (rmse_type == 0) {
        for (int i = 0; i < n; i++) {
            int l = nearest_int(iscale * x[i]);
            L[i] = (int8_t)(nmax + std::max(-nmax, std::min(nmax - 1, l)));
        }
        return 1.0f / iscale;
    }
    bool return_early = false;
    if (rmse_type < 0) { rmse_type = -rmse_type; return_early = true; }
    auto weight = [&](int i) -> float {
        switch (rmse_type) {
            case 1: return x[i] * x[i];
            case 2: return 1.0f;
            case 3: return std::fabs(x[i]);
            default: return std::sqrt(std::fabs(x[i]));
        }
    };
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = nearest_int(iscale * x[i]);
        l = std::max(-nmax, std::min(nmax - 1, l));
        L[i] = (int8_t)(l + nmax);
        float w = weight(i);
        sumlx += w * x[i] * (float)l;
        suml2 += w * (float)l * (float)l;
    }
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    if (return_early) return suml2 > 0.0f ? 0.5f * (scale + 1.0f / iscale) : 1.0f / iscale;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; is++) {
        if (is == 0) continue;
        iscale = -((float)nmax + 0.1f * (float)is) / max;
        sumlx = 0.0f;
        suml2 = 0.0f;
        for (int i = 0; i < n; i++) {
            int l = nearest_int(iscale * x[i]);
            l = std::max(-nmax, std::min(nmax - 1, l));
            float w = weight(i);
            sumlx += w * x[i] * (float)l;
            suml2 += w * (float)l * (float)l;
        }
        if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; i++) {
                int l = nearest_int(iscale * x[i]);
                L[i] = (int8_t)(nmax + std::max(-nmax, std::min(nmax - 1, l)));
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

// crates/ggml/src/quants_k.rs:2058-2130 quantize_row_q6_K_ref
static void quantize_row_q6_K_ref(const float *x, block_q6_K *y, int64_t k) {
    int8_t L[QK_K];
    float scales[QK_K / 16];
    for (int64_t i = 0; i < k / QK_K; i++) {
        const float *xb = x + i * QK_K;
        float max_scale = 0.0f, max_abs_scale = 0.0f;
        for (int ib = 0; ib < QK_K / 16; ib++) {
            float scale = make_qx_quants(16, 32, xb + 16 * ib, L + 16 * ib, 1);
            scales[ib] = scale;
            float abs_scale = std::fabs(scale);
            if (abs_scale > max_abs_scale) { max_abs_scale = abs_scale; max_scale = scale; }
        }
        if (max_abs_scale < GROUP_MAX_EPS) {
            std::memset(&y[i], 0, sizeof(block_q6_K));
            y[i].d = fp16(0.0f);
            continue;
        }
        float iscale = -128.0f / max_scale;
        uint16_t dh = fp16(1.0f / iscale);
        int8_t sb[QK_K / 16];
        for (int ib = 0; ib < QK_K / 16; ib++)
            sb[ib] = (int8_t)std::min(127, nearest_int(iscale * scales[ib]));
        for (int j = 0; j < QK_K / 16; j++) {
            float d = f32_of(dh) * (float)sb[j];
            if (d == 0.0f) continue;
            for (int ii = 0; ii < 16; ii++) {
                int l = nearest_int(xb[16 * j + ii] / d);
                L[16 * j + ii] = (int8_t)(std::max(-32, std::min(31, l)) + 32);
            }
        }
        uint8_t *ql = y[i].ql, *qh = y[i].qh;
        for (int j = 0; j < QK_K; j += 128) {
            for (int l = 0; l < 32; l++) {
                uint8_t q1 = L[j + l] & 0xF, q2 = L[j + l + 32] & 0xF;
                uint8_t q3 = L[j + l + 64] & 0xF, q4 = L[j + l + 96] & 0xF;
                ql[l] = q1 | (q3 << 4);
                ql[l + 32] = q2 | (q4 << 4);
                qh[l] = (uint8_t)((L[j + l] >> 4) | ((L[j + l + 32] >> 4) << 2) |
                                  ((L[j + l + 64] >> 4) << 4) | ((L[j + l + 96] >> 4) << 6));
            }
            ql += 64;
            qh += 32;
        }
        std::memcpy(y[i].scales, sb, sizeof(sb));
        y[i].d = dh;
    }
}

// MXFP4 weight quantizer.  The reference repo ships only the MXFP4
// *dequantizer* (crates/tools/quantize/src/rows.rs:32-33); its fixture
// parity/quants_ref_fp4.bin holds the output of upstream ggml's
// quantize_row_mxfp4_ref (ggml-quants.c at the pinned revision bd4f514db1).
// This restates that published algorithm: e = floor(log2(amax)) - 2 + 127,
// each value mapped to the nearest of the 16 codes (first minimum wins).
static void quantize_row_mxfp4_ref(const float *x, block_mxfp4 *y, int64_t k) {
    const int qk = QK_MXFP4;
    for (int64_t i = 0; i < k / qk; i++) {
        float amax = 0.0f;
        for (int j = 0; j < qk; j++) amax = std::max(amax, std::fabs(x[i * qk + j]));
        uint8_t e = amax > 0.0f ? (uint8_t)(int)(std::floor(std::log2(amax)) - 2.0f + 127.0f) : 0;
        float d = orc_e8m0_to_f32_half(e);
        auto best = [&](float v) -> uint8_t {
            int bi = 0;
            float be = std::fabs((float)KVALUES_MXFP4[0] * d - v);
            for (int c = 1; c < 16; c++) {
                float err = std::fabs((float)KVALUES_MXFP4[c] * d - v);
                if (err < be) { bi = c; be = err; }
            }
            return (uint8_t)bi;
        };
        y[i].e = e;
        for (int j = 0; j < qk / 2; j++)
            y[i].qs[j] = best(x[i * qk + j]) | (best(x[i * qk + qk / 2 + j]) << 4);
    }
}

extern "C" int orc_quantize_row(int type, const float *x, void *y, int64_t k) {
    int be = orc_block_elems(type);
    if (be == 0 || k % be != 0) return -1;
    switch (type) {
        case ORC_Q4_0: quantize_row_q4_0_ref(x, (block_q4_0 *)y, k); return 0;
        case ORC_Q8_0: quantize_row_q8_0_ref(x, (block_q8_0 *)y, k); return 0;
        case ORC_Q4_K: quantize_row_q4_K_ref(x, (block_q4_K *)y, k); return 0;
        case ORC_Q6_K: quantize_row_q6_K_ref(x, (block_q6_K *)y, k); return 0;
        case ORC_MXFP4: quantize_row_mxfp4_ref(x, (block_mxfp4 *)y, k); return 0;
        case ORC_Q8_K: orc_quantize_row_q8_K(x, y, k); return 0;
        case ORC_F16: {
            uint16_t *o = (uint16_t *)y;
            for (int64_t i = 0; i < k; i++) o[i] = fp16(x[i]);
            return 0;
        }
        case ORC_F32: std::memcpy(y, x, 4 * k); return 0;
        default: return -1;
    }
}

// ===========================================================================
// dequantizers
// ===========================================================================
extern "C" int orc_dequantize_row(int type, const void *vx, float *y, int64_t k) {
    int be = orc_block_elems(type);
    if (be == 0 || k % be != 0) return -1;
    const int64_t nb = k / be;
    switch (type) {
        case ORC_Q4_0: {  // crates/ggml/src/quants.rs:154-167
            const block_q4_0 *x = (const block_q4_0 *)vx;
            for (int64_t i = 0; i < nb; i++) {
                float d = f32_of(x[i].d);
                for (int j = 0; j < 16; j++) {
                    int x0 = (x[i].qs[j] & 0x0F) - 8, x1 = (x[i].qs[j] >> 4) - 8;
                    y[i * 32 + j] = (float)x0 * d;
                    y[i * 32 + 16 + j] = (float)x1 * d;
                }
            }
            return 0;
        }
        case ORC_Q8_0: {  // crates/ggml/src/quants.rs:364-373
            const block_q8_0 *x = (const block_q8_0 *)vx;
            for (int64_t i = 0; i < nb; i++) {
                float d = f32_of(x[i].d);
                for (int j = 0; j < 32; j++) y[i * 32 + j] = (float)x[i].qs[j] * d;
            }
            return 0;
        }
        case ORC_MXFP4: {  // crates/ggml/src/quants.rs:732-746
            const block_mxfp4 *x = (const block_mxfp4 *)vx;
            for (int64_t i = 0; i < nb; i++) {
                float d = orc_e8m0_to_f32_half(x[i].e);
                for (int j = 0; j < 16; j++) {
                    y[i * 32 + j] = (float)KVALUES_MXFP4[x[i].qs[j] & 0x0F] * d;
                    y[i * 32 + 16 + j] = (float)KVALUES_MXFP4[x[i].qs[j] >> 4] * d;
                }
            }
            return 0;
        }
        case ORC_Q4_K: {  // crates/ggml/src/quants.rs:519-547
            const block_q4_K *x = (const block_q4_K *)vx;
            for (int64_t i = 0; i < nb; i++) {
                float d = f32_of(x[i].d), min = f32_of(x[i].dmin);
                const uint8_t *q = x[i].qs;
                float *yo = y + i * QK_K;
                int is = 0;
                for (int j = 0; j < QK_K; j += 64) {
                    uint8_t sc, m;
                    get_scale_min_k4(is, x[i].scales, &sc, &m);
                    float d1 = d * (float)sc, m1 = min * (float)m;
                    get_scale_min_k4(is + 1, x[i].scales, &sc, &m);
                    float d2 = d * (float)sc, m2 = min * (float)m;
                    for (int l = 0; l < 32; l++) yo[l] = d1 * (float)(q[l] & 0xF) - m1;
                    for (int l = 0; l < 32; l++) yo[32 + l] = d2 * (float)(q[l] >> 4) - m2;
                    yo += 64;
                    q += 32;
                    is += 2;
                }
            }
            return 0;
        }
        case ORC_Q6_K: {  // crates/ggml/src/quants.rs:585-612
            const block_q6_K *x = (const block_q6_K *)vx;
            for (int64_t i = 0; i < nb; i++) {
                float d = f32_of(x[i].d);
                const uint8_t *ql = x[i].ql, *qh = x[i].qh;
                const int8_t *sc = x[i].scales;
                float *yo = y + i * QK_K;
                for (int n = 0; n < QK_K; n += 128) {
                    for (int l = 0; l < 32; l++) {
                        int is = l / 16;
                        int q1 = (int)(int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                        int q2 = (int)(int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                        int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                        int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                        yo[l] = d * (float)sc[is + 0] * (float)q1;
                        yo[l + 32] = d * (float)sc[is + 2] * (float)q2;
                        yo[l + 64] = d * (float)sc[is + 4] * (float)q3;
                        yo[l + 96] = d * (float)sc[is + 6] * (float)q4;
                    }
                    yo += 128;
                    ql += 64;
                    qh += 32;
                    sc += 8;
                }
            }
            return 0;
        }
        case ORC_Q8_K: {
            const block_q8_K *x = (const block_q8_K *)vx;
            for (int64_t i = 0; i < nb; i++)
                for (int j = 0; j < QK_K; j++) y[i * QK_K + j] = x[i].d * (float)x[i].qs[j];
            return 0;
        }
        case ORC_F16: {
            const uint16_t *x = (const uint16_t *)vx;
            for (int64_t i = 0; i < k; i++) y[i] = f32_of(x[i]);
            return 0;
        }
        case ORC_F32: std::memcpy(y, vx, 4 * k); return 0;
        default: return -1;
    }
}

// ===========================================================================
// activation quantizers
// ===========================================================================

// A1 — crates/ggml/src/quants.rs:331-362 quantize_row_q8_0 (runtime form:
// id = 127/amax, round-to-nearest-even, INT_MIN lanes saturate to -128)
extern "C" void orc_quantize_row_q8_0(const float *x, void *vy, int64_t k) {
    block_q8_0 *y = (block_q8_0 *)vy;
    for (int64_t i = 0; i < k / QK8_0; i++) {
        float amax = 0.0f;
        for (int j = 0; j < QK8_0; j++) amax = std::max(amax, std::fabs(x[i * QK8_0 + j]));
        const float d = amax / 127.0f;
        const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
        for (int j = 0; j < QK8_0; j++) {
            float r = std::nearbyint(x[i * QK8_0 + j] * id);
            if (std::isnan(r) || std::fabs(r) >= 2147483648.0f) {
                y[i].qs[j] = INT8_MIN;
            } else {
                y[i].qs[j] = (int8_t)std::max(-128.0f, std::min(127.0f, r));
            }
        }
        y[i].d = fp16(d);
    }
}

// A2 — crates/ggml/src/quants.rs:615-654 quantize_row_q8_K(_ref): the first
// element of largest magnitude fixes the sign of d.
extern "C" void orc_quantize_row_q8_K(const float *x, void *vy, int64_t k) {
    block_q8_K *y = (block_q8_K *)vy;
    for (int64_t i = 0; i < k / QK_K; i++) {
        const float *xb = x + i * QK_K;
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < QK_K; j++) {
            float ax = std::fabs(xb[j]);
            if (ax > amax) { amax = ax; max = xb[j]; }
        }
        if (amax == 0.0f) {
            std::memset(&y[i], 0, sizeof(block_q8_K));
            continue;
        }
        const float iscale = -127.0f / max;
        for (int j = 0; j < QK_K; j++) {
            int v = nearest_int(iscale * xb[j]);
            y[i].qs[j] = (int8_t)std::min(127, v);
        }
        for (int j = 0; j < QK_K / 16; j++) {
            int sum = 0;
            for (int ii = 0; ii < 16; ii++) sum += y[i].qs[j * 16 + ii];
            y[i].bsums[j] = (int16_t)sum;
        }
        y[i].d = 1.0f / iscale;
    }
}

// A3 — crates/ggml/src/repack.rs:1561-1606 quantize_mat_q8_K_4x8.
// block_q8_Kx4 = d[4] f32 | qs[1024] | bsums[64] i16 (1168 bytes).
extern "C" void orc_quantize_mat_q8_K_4x8(const float *x, int64_t k, int64_t n_rows, void *vout) {
    uint8_t *out = (uint8_t *)vout;
    const int64_t nb = k / QK_K;
    const size_t TILE = 1168;
    for (int64_t r4 = 0; r4 < n_rows / 4; r4++) {
        const float *rows = x + r4 * 4 * k;
        for (int64_t ib = 0; ib < nb; ib++) {
            uint8_t *blk = out + (r4 * nb + ib) * TILE;
            float *d = (float *)blk;
            int8_t *qs = (int8_t *)(blk + 16);
            int16_t *bsums = (int16_t *)(blk + 16 + 1024);
            for (int r = 0; r < 4; r++) {
                const float *xb = rows + r * k + ib * QK_K;
                float max_abs = 0.0f;
                for (int j = 0; j < QK_K; j++) {
                    float a = std::fabs(xb[j]);
                    if (a > max_abs) max_abs = a;
                }
                const float iscale = max_abs != 0.0f ? 127.0f / max_abs : 0.0f;
                d[r] = max_abs != 0.0f ? 1.0f / iscale : 0.0f;
                for (int el = 0; el < QK_K; el++) {
                    float q = std::nearbyint(iscale * xb[el]);
                    q = std::max(-128.0f, std::min(127.0f, q));
                    qs[(el / 8) * 32 + r * 8 + el % 8] = (int8_t)q;
                }
            }
            std::memset(bsums, 0, 128);
            for (int r = 0; r < 4; r++)
                for (int el = 0; el < QK_K; el++) {
                    int q = qs[(el / 8) * 32 + r * 8 + el % 8];
                    int idx = 16 * (el / 64) + 4 * r + (el / 16) % 4;
                    bsums[idx] = (int16_t)(bsums[idx] + q);
                }
        }
    }
}

// A4 — crates/ggml/src/repack.rs:247-274 quantize_mat_q8_0_4x8.
// block_q8_0x4 = d[4] f16 | qs[128] interleaved by 8 (136 bytes).
extern "C" void orc_quantize_mat_q8_0_4x8(const float *x, int64_t k, int64_t n_rows, void *vout) {
    uint8_t *out = (uint8_t *)vout;
    const int64_t nb = k / QK8_0;
    const int interleave = 8;
    std::vector<block_q8_0> q8(4 * nb);
    for (int64_t r = 0; r < n_rows / 4; r++) {
        orc_quantize_row_q8_0(x + r * 4 * k, q8.data(), 4 * k);
        for (int64_t ib = 0; ib < nb; ib++) {
            uint8_t *blk = out + (r * nb + ib) * 136;
            for (int rr = 0; rr < 4; rr++) std::memcpy(blk + 2 * rr, &q8[rr * nb + ib].d, 2);
            for (int j = 0; j < QK8_0 * 4; j++) {
                int src_id = (j % (4 * interleave)) / interleave;
                int src_offset = (j / (4 * interleave)) * interleave + (j % interleave);
                blk[8 + j] = (uint8_t)q8[src_id * nb + ib].qs[src_offset];
            }
        }
    }
}

// ===========================================================================
// 8x8 interleaved weight layouts
// ===========================================================================

// crates/ggml/src/repack.rs:1351-1423 make_block_q4_Kx8
static void make_block_q4_Kx8(const block_q4_K *in8, uint8_t *out) {
    for (int i = 0; i < 8; i++) {
        std::memcpy(out + 2 * i, &in8[i].d, 2);
        std::memcpy(out + 16 + 2 * i, &in8[i].dmin, 2);
    }
    for (int i = 0; i < 128; i++) {
        int src_id = i % 8, src_offset = (i / 8) * 8;
        std::memcpy(out + 128 + i * 8, in8[src_id].qs + src_offset, 8);
    }
    uint8_t *scales = out + 32;
    for (int half = 0; half < 2; half++) {
        for (int i = 0; i < 4; i++) {
            uint8_t s[8], m[8];
            for (int j = 0; j < 8; j++) {
                const uint8_t *sc = in8[j].scales;
                if (half == 0) {
                    s[j] = sc[i] & 63;
                    m[j] = sc[i + 4] & 63;
                } else {
                    s[j] = ((sc[i] & 192) >> 2) | (sc[i + 8] & 15);
                    m[j] = ((sc[i + 4] & 192) >> 2) | ((sc[i + 8] & 240) >> 4);
                }
            }
            int sb = half * 4 + i;
            int g = sb < 4 ? 12 * sb : 12 * (sb - 4) + 48;
            for (int t = 0; t < 4; t++) {
                scales[g + t] = (s[t] & 63) + ((s[4 + t] & 48) << 2);
                scales[g + 4 + t] = (m[t] & 63) + ((m[4 + t] & 48) << 2);
                scales[g + 8 + t] = (s[4 + t] & 15) + ((m[4 + t] & 15) << 4);
            }
        }
    }
}

extern "C" int orc_repack_8x8(int type, const void *vsrc, int64_t nrows, int64_t k, void *vdst) {
    const uint8_t *src = (const uint8_t *)vsrc;
    uint8_t *dst = (uint8_t *)vdst;
    if (nrows % 8 != 0) return -1;
    if (type == ORC_Q4_K) {  // crates/ggml/src/repack.rs:1435-1468
        if (k % QK_K) return -1;
        const int64_t nb = k / QK_K;
        for (int64_t g = 0; g < nrows / 8; g++) {
            const block_q4_K *sg = (const block_q4_K *)(src + g * 8 * nb * 144);
            uint8_t *dg = dst + g * 8 * nb * 144;
            for (int64_t x = 0; x < nb; x++) {
                block_q4_K tmp[8];
                for (int i = 0; i < 8; i++) tmp[i] = sg[x + i * nb];
                make_block_q4_Kx8(tmp, dg + x * 1152);
            }
        }
        return 0;
    }
    if (type == ORC_Q4_0 || type == ORC_MXFP4) {
        // crates/ggml/src/repack.rs:3235-3282 (Q4_0, bytes ^ 0x88) and :138-189 (MXFP4)
        if (k % 32) return -1;
        const int64_t nb = k / 32;
        const int hdr = type == ORC_Q4_0 ? 2 : 1;
        const int bsz = hdr + 16, tile = 8 * bsz;
        for (int64_t g = 0; g < nrows / 8; g++) {
            const uint8_t *sg = src + g * 8 * nb * bsz;
            uint8_t *dg = dst + g * 8 * nb * bsz;
            for (int64_t x = 0; x < nb; x++) {
                uint8_t *t = dg + x * tile;
                for (int i = 0; i < 8; i++)
                    std::memcpy(t + hdr * i, sg + (i * nb + x) * bsz, hdr);
                for (int i = 0; i < 16; i++) {
                    int src_id = i % 8, src_offset = (i / 8) * 8;
                    const uint8_t *s = sg + (src_id * nb + x) * bsz + hdr + src_offset;
                    uint8_t *o = t + 8 * hdr + i * 8;
                    for (int b = 0; b < 8; b++) o[b] = type == ORC_Q4_0 ? (s[b] ^ 0x88) : s[b];
                }
            }
        }
        return 0;
    }
    return -1;
}
