// CPU oracle, part 3: FLASH_ATTN_EXT over an F16 KV cache.
//
// TEST INFRASTRUCTURE ONLY (see oracle.h).  Scalar restatement of
// crates/ggml/src/flash_attn.rs (and the f16 dot of vec_dot.rs) for q F32,
// k/v F16, mask F16, batch (ne3) 1:
//   one_chunk  flash_attn.rs:482-736   online softmax per row, F16 V keeps the
//              accumulator in f16 with one rounding per scale / mad
//   split-KV   flash_attn.rs:744-859   n_chunks partial rows merged in order
//   tiled      flash_attn.rs:1103-1361 64x64 tiles, f32 FMA chains, v_expf
// Layouts: q element (d, t, h) at q + t*q_nb1 + h*q_nb2 (bytes) + 4d; k/v row
// (pos, hkv) at k + pos*k_nb1 + hkv*k_nb2; mask row t at mask + t*mask_nb1;
// dst[(t*H + h)*DV + d] (ggml dst ne = [DV, H, T]).
#include "oracle.h"

#include <omp.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

namespace {

inline float h2f(uint16_t h) { return orc_f16_to_f32(h); }
inline uint16_t f2h(float f) { return orc_f32_to_f16(f); }
const float NEG_INF = -std::numeric_limits<float>::infinity();

inline const uint8_t *bp(const void *p) { return (const uint8_t *)p; }

// crates/ggml/src/vec_dot.rs:1893-1903 reduce_add16
float reduce_add16(const float *x) {
    float t[16];
    std::memcpy(t, x, sizeof(t));
    for (int half = 8; half >= 1; half >>= 1)
        for (int i = 0; i < half; i++) t[i] += t[i + half];
    return t[0];
}

// crates/ggml/src/vec_dot.rs:1982-2019 vec_dot_f16_c: 4 x 16 f32 lanes, fma(y, x, s)
float vec_dot_f16(int64_t n, const uint16_t *x, const uint16_t *y) {
    const int64_t np = n & ~(int64_t)63;
    float sum[4][16] = {{0}};
    int64_t i = 0;
    for (; i < np; i += 64)
        for (int j = 0; j < 4; j++)
            for (int l = 0; l < 16; l++) {
                int k = j * 16 + l;
                sum[j][l] = fmaf(h2f(y[i + k]), h2f(x[i + k]), sum[j][l]);
            }
    float a[16], b[16];
    for (int l = 0; l < 16; l++) a[l] = sum[0][l] + sum[2][l];
    for (int l = 0; l < 16; l++) b[l] = sum[1][l] + sum[3][l];
    for (int l = 0; l < 16; l++) a[l] += b[l];
    double res = (double)reduce_add16(a);
    for (; i < n; i++) res += (double)(h2f(x[i]) * h2f(y[i]));
    return (float)res;
}

// crates/ggml/src/flash_attn.rs:356-377: ALiBi slope and the softcap pre-division
float slope_of(const OrcFlashArgs *a, int64_t h) {
    if (a->max_bias <= 0.0f) return 1.0f;
    const uint32_t nl2 = 1u << (uint32_t)std::floor(std::log2((double)a->H));
    const float m0 = std::pow(2.0f, -a->max_bias / (float)nl2);
    const float m1 = std::pow(2.0f, -(a->max_bias / 2.0f) / (float)nl2);
    if ((uint32_t)h < nl2) return __builtin_powif(m0, (int)h + 1);
    return __builtin_powif(m1, (int)(2 * ((uint32_t)h - nl2) + 1));
}
float kq_scale_of(const OrcFlashArgs *a) {
    return a->logit_softcap != 0.0f ? a->scale / a->logit_softcap : a->scale;
}

// crates/ggml/src/flash_attn.rs:482-694 attn_row: (t, h) over KV [ic0, ic1);
// unnormalized accumulator in vkq (f32 copy of the f16 accumulator), returns M, S.
void attn_row(const OrcFlashArgs *a, int64_t t, int64_t h, int64_t ic0, int64_t ic1, float *vkq, float *M_out,
              float *S_out) {
    const int64_t dk = a->dk, dv = a->dv;
    const int64_t hkv = h / (a->H / a->H_kv);
    const float slope = slope_of(a, h);
    const float kq_scale = kq_scale_of(a);
    const float softcap = a->logit_softcap;
    float S = 0.0f, M = NEG_INF;
    std::vector<uint16_t> vkq16(dv, 0), q16(dk);
    const float *q = (const float *)(bp(a->q) + t * a->q_nb1 + h * a->q_nb2);
    for (int64_t d = 0; d < dk; d++) q16[d] = f2h(q[d]);
    const uint8_t *kb = bp(a->k) + hkv * a->k_nb2;
    const uint8_t *vb = bp(a->v) + hkv * a->v_nb2;
    const uint16_t *mrow = a->mask ? (const uint16_t *)(bp(a->mask) + t * a->mask_nb1) : nullptr;
    for (int64_t ic = ic0; ic < ic1; ic++) {
        const float mv = mrow ? slope * h2f(mrow[ic]) : 0.0f;
        if (mv == NEG_INF) continue;
        float s = vec_dot_f16(dk, (const uint16_t *)(kb + ic * a->k_nb1), q16.data()) * kq_scale;
        if (softcap != 0.0f) s = softcap * std::tanh(s);
        s += mv;
        const float Mold = M;
        float ms = 1.0f, vs = 1.0f;
        const uint16_t *vrow = (const uint16_t *)(vb + ic * a->v_nb1);
        if (s > M) {
            M = s;
            ms = std::exp(Mold - M);
            for (int64_t d = 0; d < dv; d++) vkq16[d] = f2h(h2f(vkq16[d]) * ms);
        } else {
            vs = std::exp(s - M);
        }
        for (int64_t d = 0; d < dv; d++) vkq16[d] = f2h(fmaf(h2f(vrow[d]), vs, h2f(vkq16[d])));
        S = fmaf(S, ms, vs);
    }
    for (int64_t d = 0; d < dv; d++) vkq[d] = h2f(vkq16[d]);
    if (a->sinks && ic0 == 0) {
        const float sh = a->sinks[h];
        float ms = 1.0f, vs = 1.0f;
        if (sh > M) {
            ms = std::exp(M - sh);
            M = sh;
            for (int64_t d = 0; d < dv; d++) vkq[d] *= ms;
        } else {
            vs = std::exp(sh - M);
        }
        S = S * ms + vs;  // two roundings here, unlike the loop (flash_attn.rs:676-688)
    }
    *M_out = M;
    *S_out = S;
}

void write_normalized(const OrcFlashArgs *a, int64_t t, int64_t h, float *vkq, float S) {
    const float s_inv = S == 0.0f ? 0.0f : 1.0f / S;
    float *o = a->dst + (t * a->H + h) * a->dv;
    for (int64_t d = 0; d < a->dv; d++) o[d] = vkq[d] * s_inv;
}

// crates/ggml/src/flash_attn.rs:728-736
void one_chunk(const OrcFlashArgs *a) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t h = 0; h < a->H; h++)
        for (int64_t t = 0; t < a->T; t++) {
            std::vector<float> vkq(a->dv);
            float M, S;
            attn_row(a, t, h, 0, a->n_kv, vkq.data(), &M, &S);
            write_normalized(a, t, h, vkq.data(), S);
        }
}

// crates/ggml/src/flash_attn.rs:744-859 split_kv + reduce_partials
void split_kv(const OrcFlashArgs *a, int n_chunks) {
    const int64_t dv = a->dv, H = a->H, n_kv = a->n_kv;
    const int64_t chunk = (n_kv + n_chunks - 1) / n_chunks;
    const int64_t psz = 2 + dv;
    std::vector<float> part((size_t)H * n_chunks * psz, 0.0f);
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int c = 0; c < n_chunks; c++)
        for (int64_t h = 0; h < H; h++) {
            float *p = &part[((size_t)h * n_chunks + c) * psz];
            const int64_t ic0 = c * chunk, ic1 = std::min(ic0 + chunk, n_kv);
            if (ic0 >= n_kv) {
                p[0] = NEG_INF;
                p[1] = 0.0f;
                continue;
            }
            attn_row(a, 0, h, ic0, ic1, p + 2, &p[0], &p[1]);
        }
    for (int64_t h = 0; h < H; h++) {
        std::vector<float> fin(dv, 0.0f);
        float Mf = NEG_INF, Sf = 0.0f;
        for (int c = 0; c < n_chunks; c++) {
            if ((int64_t)c * chunk >= n_kv) continue;
            const float *p = &part[((size_t)h * n_chunks + c) * psz];
            const float Mc = p[0], Sc = p[1];
            if (Sc == 0.0f) continue;
            const float Mn = std::max(Mf, Mc);
            const float so = std::exp(Mf - Mn), sn = std::exp(Mc - Mn);
            for (int64_t d = 0; d < dv; d++) fin[d] = fmaf(fin[d], so, p[2 + d] * sn);
            Sf = fmaf(Sf, so, Sc * sn);
            Mf = Mn;
        }
        if (Sf != 0.0f) {
            const float s_inv = 1.0f / Sf;
            for (int64_t d = 0; d < dv; d++) fin[d] *= s_inv;
        }
        std::memcpy(a->dst + h * dv, fin.data(), dv * 4);
    }
}

// crates/ggml/src/flash_attn.rs:948-975 v_expf (one lane of the AVX512 ggml_v_expf)
inline float bits_f(uint32_t b) {
    float f;
    std::memcpy(&f, &b, 4);
    return f;
}
float v_expf(float x) {
    const float R = bits_f(0x4b400000), LOG2E = bits_f(0x3fb8aa3b), C1 = bits_f(0x35bfbe8e), C2 = bits_f(0x3f317200);
    const float P1 = bits_f(0x3c072010), P2 = bits_f(0x3d2b9f17), P3 = bits_f(0x3e2aaf33), P4 = bits_f(0x3efffedb);
    const float P5 = bits_f(0x3f7ffff6);
    const float z = fmaf(x, LOG2E, R);
    const float n = z - R;
    const float b = fmaf(n, -C1, fmaf(n, -C2, x));
    const float u = b * b;
    const float j = fmaf(fmaf(fmaf(b, P1, P2), u, fmaf(b, P3, P4)), u, fmaf(b, P5, 1.0f));
    if (std::fabs(n) > 192.0f) return n <= 0.0f ? 0.0f : std::numeric_limits<float>::infinity();
    return (float)((double)j * std::ldexp(1.0, (int)n));
}
// crates/ggml/src/flash_attn.rs:997-1005 (_mm512_reduce_add_ps as gcc emits it)
float reduce_add_ps(const float *v) {
    float t3[8];
    for (int j = 0; j < 8; j++) t3[j] = v[8 + j] + v[j];
    const float t6[4] = {t3[4] + t3[0], t3[5] + t3[1], t3[6] + t3[2], t3[7] + t3[3]};
    return (t6[0] + t6[2]) + (t6[1] + t6[3]);
}
// crates/ggml/src/flash_attn.rs:1027-1049 vec_soft_max_f32 in place, f64 sum
double soft_max_inplace(float *y, int n, float max) {
    int i = 0;
    double sum = 0.0;
    for (; i + 15 < n; i += 16) {
        float v[16];
        for (int j = 0; j < 16; j++) v[j] = v_expf(y[i + j] - max);
        std::memcpy(y + i, v, sizeof(v));
        sum += (double)reduce_add_ps(v);
    }
    for (; i < n; i++) {
        const float val = std::exp(y[i] - max);
        sum += (double)val;
        y[i] = val;
    }
    return sum;
}
// crates/ggml/src/flash_attn.rs:1069-1079 simd_gemm: one fma chain per element, kk ascending
void gemm_acc(float *c, const float *a, const float *b, int m, int k, int n) {
    for (int i = 0; i < m; i++)
        for (int kk = 0; kk < k; kk++) {
            const float av = a[i * k + kk];
            const float *br = b + (size_t)kk * n;
            float *cr = c + (size_t)i * n;
            for (int x = 0; x < n; x++) cr[x] = fmaf(av, br[x], cr[x]);
        }
}

// crates/ggml/src/flash_attn.rs:1111-1361 tiled_impl, one (head, 64-row) tile
void tiled_tile(const OrcFlashArgs *a, int64_t h, int64_t t0) {
    constexpr int QT = 64, KT = 64;
    const int dk = (int)a->dk, dv = (int)a->dv;
    const int64_t n_kv = a->n_kv;
    const int tile_rows = (int)std::min<int64_t>(QT, a->T - t0);
    const int64_t hkv = h / (a->H / a->H_kv);
    const float slope = slope_of(a, h), kq_scale = kq_scale_of(a), softcap = a->logit_softcap;
    std::vector<float> qf((size_t)QT * dk, 0.0f), kq((size_t)QT * KT), mask32((size_t)QT * KT, 0.0f);
    std::vector<float> vkq((size_t)QT * dv, 0.0f), v32((size_t)KT * dv, 0.0f), kf((size_t)KT * dk, 0.0f);
    float S[QT], M[QT];
    for (int i = 0; i < QT; i++) { S[i] = 0.0f; M[i] = NEG_INF; }
    for (int tq = 0; tq < tile_rows; tq++)
        std::memcpy(&qf[(size_t)tq * dk], bp(a->q) + (t0 + tq) * a->q_nb1 + h * a->q_nb2, dk * 4);
    const uint8_t *kb = bp(a->k) + hkv * a->k_nb2;
    const uint8_t *vb = bp(a->v) + hkv * a->v_nb2;
    for (int64_t ic = 0; ic < n_kv; ic += KT) {
        const int kv_tile = (int)std::min<int64_t>(KT, n_kv - ic);
        if (a->mask) {
            bool can_skip = true;
            for (int tq = 0; tq < tile_rows; tq++) {
                const uint16_t *mrow = (const uint16_t *)(bp(a->mask) + (t0 + tq) * a->mask_nb1);
                for (int tk = 0; tk < kv_tile; tk++) {
                    const float mv = slope * h2f(mrow[ic + tk]);
                    mask32[tq * KT + tk] = mv;
                    if (mv != NEG_INF) can_skip = false;
                }
                for (int tk = kv_tile; tk < KT; tk++) mask32[tq * KT + tk] = NEG_INF;
            }
            if (can_skip) continue;
        }
        for (int tk = 0; tk < kv_tile; tk++) {
            const uint16_t *krow = (const uint16_t *)(kb + (ic + tk) * a->k_nb1);
            for (int d = 0; d < dk; d++) kf[(size_t)d * KT + tk] = h2f(krow[d]);
        }
        std::fill(kq.begin(), kq.end(), 0.0f);
        gemm_acc(kq.data(), qf.data(), kf.data(), QT, dk, KT);
        for (auto &x : kq) x *= kq_scale;
        if (softcap != 0.0f)
            for (auto &x : kq) x = softcap * std::tanh(x);
        if (kv_tile < KT)
            for (int tq = 0; tq < QT; tq++)
                for (int tk = kv_tile; tk < KT; tk++) kq[tq * KT + tk] = NEG_INF;
        if (a->mask)
            for (int i = 0; i < tile_rows * KT; i++) kq[i] += mask32[i];
        bool skip[QT];
        for (int tq = 0; tq < QT; tq++) {
            skip[tq] = false;
            float *row = &kq[(size_t)tq * KT];
            float tmax = NEG_INF;
            for (int i = 0; i < KT; i++) tmax = tmax > row[i] ? tmax : row[i];
            if (tmax == NEG_INF) { skip[tq] = true; continue; }
            const float m_old = M[tq];
            const float m_new = m_old > tmax ? m_old : tmax;
            if (m_new > m_old) {
                const float ms = std::exp(m_old - m_new);
                for (int d = 0; d < dv; d++) vkq[(size_t)tq * dv + d] *= ms;
                S[tq] *= ms;
            }
            M[tq] = m_new;
            const double sum = soft_max_inplace(row, KT, m_new);
            S[tq] = (float)((double)S[tq] + sum);
        }
        for (int tk = 0; tk < kv_tile; tk++) {
            const uint16_t *vrow = (const uint16_t *)(vb + (ic + tk) * a->v_nb1);
            for (int d = 0; d < dv; d++) v32[(size_t)tk * dv + d] = h2f(vrow[d]);
        }
        for (int tq = 0; tq < QT; tq++)
            if (skip[tq]) std::fill(kq.begin() + (size_t)tq * KT, kq.begin() + (size_t)(tq + 1) * KT, 0.0f);
        gemm_acc(vkq.data(), kq.data(), v32.data(), QT, KT, dv);
    }
    if (a->sinks) {
        const float sv = a->sinks[h];
        for (int tq = 0; tq < tile_rows; tq++) {
            float ms = 1.0f, vs = 1.0f;
            if (sv > M[tq]) {
                ms = std::exp(M[tq] - sv);
                for (int d = 0; d < dv; d++) vkq[(size_t)tq * dv + d] *= ms;
            } else {
                vs = std::exp(sv - M[tq]);
            }
            S[tq] = fmaf(S[tq], ms, vs);
        }
    }
    for (int tq = 0; tq < tile_rows; tq++) {
        const float s_inv = S[tq] == 0.0f ? 0.0f : 1.0f / S[tq];
        float *o = a->dst + ((t0 + tq) * a->H + h) * dv;
        for (int d = 0; d < dv; d++) o[d] = vkq[(size_t)tq * dv + d] * s_inv;
    }
}

void tiled(const OrcFlashArgs *a) {
    const int64_t nt = (a->T + 63) / 64;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int64_t h = 0; h < a->H; h++)
        for (int64_t it = 0; it < nt; it++) tiled_tile(a, h, it * 64);
}

}  // namespace

// Dispatch of crates/ggml/src/flash_attn.rs:907-939: split-KV for a single
// query row with n_kv >= 512, tiled from 64 query rows on, else one_chunk.
// Returns the mode taken (1 one_chunk, 2 split-KV, 3 tiled) or -1.
// one lane of the 16-wide polynomial exp, for the glue ops that share it (silu)
extern "C" float orc_v_expf(float x) { return v_expf(x); }

extern "C" int orc_flash_attn_ext(const OrcFlashArgs *a) {
    if (!a || a->dk <= 0 || a->dv <= 0 || a->H_kv <= 0 || a->H % a->H_kv != 0) return -1;
    if (a->max_bias > 0.0f && !a->mask) return -1;
    if (a->n_threads > 0) omp_set_num_threads(a->n_threads);
    int mode = a->mode;
    if (mode == 0) mode = (a->T == 1 && a->n_kv >= 512) ? 2 : (a->T >= 64 ? 3 : 1);
    if (mode == 2) {
        if (a->T != 1 || a->n_chunks < 1) return -1;
        split_kv(a, a->n_chunks);
    } else if (mode == 3) {
        tiled(a);
    } else if (mode == 1) {
        one_chunk(a);
    } else {
        return -1;
    }
    return mode;
}
