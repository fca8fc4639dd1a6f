// CPU oracle, part 4: the f32 glue ops that sit between the quantized mat-muls of a decoder
// layer, and a Llama forward pass assembled from them.
//
// TEST INFRASTRUCTURE ONLY (see oracle.h).  Each function restates the reference's CPU
// arithmetic and names the file:line it follows.  cosf / sinf / powf / logf / expf are the host
// libm's, exactly as the reference calls them.
#include <cmath>
#include <cstring>
#include <limits>
#include <unordered_map>
#include <vector>

#include "oracle.h"

extern "C" float orc_v_expf(float x);

extern "C" {

// crates/ggml/src/compute.rs:2634-2683 forward_rms_norm: f64 running sum of the f32 squares in
// element order, mean narrowed to f32, scale = 1/sqrt(mean + eps), one rounded multiply per lane.
void orc_rms_norm(const float *x, float *y, int64_t ne0, int64_t nrows, float eps) {
    for (int64_t r = 0; r < nrows; r++) {
        const float *xr = x + r * ne0;
        float *yr = y + r * ne0;
        double sum = 0.0;
        for (int64_t i = 0; i < ne0; i++) sum += (double)(xr[i] * xr[i]);
        const float mean = (float)(sum / (double)ne0);
        const float scale = 1.0f / std::sqrt(mean + eps);
        for (int64_t i = 0; i < ne0; i++) yr[i] = xr[i] * scale;
    }
}

// crates/ggml/src/compute.rs:1174-1330 forward_bin_op, F32 x F32 -> F32: row r of b is
// r % b_rows, element i of it is i % b_ne0; one rounded op per element.
void orc_add(const float *a, const float *b, float *y, int64_t ne0, int64_t nrows, int64_t b_ne0, int64_t b_rows) {
    for (int64_t r = 0; r < nrows; r++)
        for (int64_t i = 0; i < ne0; i++) y[r * ne0 + i] = a[r * ne0 + i] + b[(r % b_rows) * b_ne0 + i % b_ne0];
}
void orc_mul(const float *a, const float *b, float *y, int64_t ne0, int64_t nrows, int64_t b_ne0, int64_t b_rows) {
    for (int64_t r = 0; r < nrows; r++)
        for (int64_t i = 0; i < ne0; i++) y[r * ne0 + i] = a[r * ne0 + i] * b[(r % b_rows) * b_ne0 + i % b_ne0];
}

// crates/ggml/src/ops.rs:267 ggml_silu_scalar_f32 (libm expf)
static inline float silu_scalar(float x) { return x / (1.0f + std::exp(-x)); }
// crates/ggml/src/simd_x86.rs:1012-1020 v_silu_16, one lane: x / (1 + v_expf(0 - x))
static inline float silu_wide_lane(float x) { return x / (1.0f + orc_v_expf(0.0f - x)); }

// crates/ggml/src/simd_x86.rs:1028-1054 vec_silu_f32 per row: on an AVX512F+DQ host (wide != 0)
// whole 16-lane chunks take the polynomial and the tail takes libm expf; otherwise libm throughout.
void orc_silu(const float *x, float *y, int64_t ne0, int64_t nrows, int wide) {
    for (int64_t r = 0; r < nrows; r++) {
        const float *xr = x + r * ne0;
        float *yr = y + r * ne0;
        int64_t i = 0;
        if (wide)
            for (; i + 16 <= ne0; i += 16)
                for (int j = 0; j < 16; j++) yr[i + j] = silu_wide_lane(xr[i + j]);
        for (; i < ne0; i++) yr[i] = silu_scalar(xr[i]);
    }
}
// crates/ggml/src/simd_x86.rs:1060-1085 vec_swiglu_f32: silu(x) * g with the same chunk / tail split
void orc_swiglu(const float *x, const float *g, float *y, int64_t ne0, int64_t nrows, int wide) {
    for (int64_t r = 0; r < nrows; r++) {
        const float *xr = x + r * ne0, *gr = g + r * ne0;
        float *yr = y + r * ne0;
        int64_t i = 0;
        if (wide)
            for (; i + 16 <= ne0; i += 16)
                for (int j = 0; j < 16; j++) yr[i + j] = silu_wide_lane(xr[i + j]) * gr[i + j];
        for (; i < ne0; i++) yr[i] = silu_scalar(xr[i]) * gr[i];
    }
}

// crates/ggml/src/compute.rs:3513-3517 rope_yarn_ramp
static float rope_yarn_ramp(float low, float high, int64_t i0) {
    const float y = ((float)(i0 / 2) - low) / std::fmax(0.001f, high - low);
    return 1.0f - std::fmin(1.0f, std::fmax(0.0f, y));
}
// crates/ggml/src/compute.rs:3627-3635 rope_yarn_corr_dims
static void rope_corr_dims(int n_dims, int n_ctx_orig, float freq_base, float beta_fast, float beta_slow, float dims[2]) {
    auto corr_dim = [&](float n_rot) {
        return (float)n_dims * std::log((float)n_ctx_orig / (n_rot * 2.0f * 3.14159265358979323846f)) / (2.0f * std::log(freq_base));
    };
    const float start = std::floor(corr_dim(beta_fast));
    const float end = std::ceil(corr_dim(beta_slow));
    dims[0] = std::fmax(0.0f, start);
    dims[1] = std::fmin((float)(n_dims - 1), end);
}

// The (cos, sin) cache of one position — crates/ggml/src/compute.rs:3520-3566 rope_yarn +
// rope_cache_init: theta starts at the position, is multiplied by theta_scale once per pair
// over the whole row, and each pair takes cosf/sinf of theta/ff (times freq_scale, yarn-mixed
// when ext_factor != 0) scaled by the attention factor.  cache: ne0 floats, (cos, sin) pairs.
void orc_rope_cache(int32_t pos, int64_t ne0, const float *freq_factors, int n_dims, int n_ctx_orig, float freq_base,
                    float freq_scale, float ext_factor, float attn_factor, float beta_fast, float beta_slow, float *cache) {
    const float theta_scale = std::pow(freq_base, -2.0f / (float)n_dims);
    float corr[2];
    rope_corr_dims(n_dims, n_ctx_orig, freq_base, beta_fast, beta_slow, corr);
    float theta = (float)pos;
    for (int64_t i0 = 0; i0 < ne0; i0 += 2) {
        const float ff = freq_factors ? freq_factors[i0 / 2] : 1.0f;
        const float theta_extrap = theta / ff;
        const float theta_interp = freq_scale * theta_extrap;
        float th = theta_interp, mscale = attn_factor;
        if (ext_factor != 0.0f) {
            const float ramp_mix = rope_yarn_ramp(corr[0], corr[1], i0) * ext_factor;
            th = theta_interp * (1.0f - ramp_mix) + theta_extrap * ramp_mix;
            mscale *= 1.0f + 0.1f * std::log(1.0f / freq_scale);
        }
        cache[i0] = std::cos(th) * mscale;
        cache[i0 + 1] = std::sin(th) * mscale;
        theta *= theta_scale;
    }
}

// crates/ggml/src/compute.rs:3663-3800 forward_rope, F32, mode 0 (NORMAL: adjacent pairs) and
// mode 2 (NEOX: pairs n_dims/2 apart); x, y: [n_tok][n_head][ne0]; channels past n_dims copy.
// rotate_pairs_f32: out0 = fma(x0, cos, -(x1*sin)), out1 = fma(x0, sin, x1*cos).
int orc_rope(const float *x, float *y, int64_t ne0, int64_t n_head, int64_t n_tok, const int32_t *pos,
             const float *freq_factors, int n_dims, int mode, int n_ctx_orig, float freq_base, float freq_scale,
             float ext_factor, float attn_factor, float beta_fast, float beta_slow) {
    if ((mode != 0 && mode != 2) || n_dims > ne0 || n_dims % 2) return -1;
    std::vector<float> cache(ne0);
    for (int64_t t = 0; t < n_tok; t++) {
        orc_rope_cache(pos[t], ne0, freq_factors, n_dims, n_ctx_orig, freq_base, freq_scale, ext_factor, attn_factor,
                       beta_fast, beta_slow, cache.data());
        for (int64_t h = 0; h < n_head; h++) {
            const float *src = x + (t * n_head + h) * ne0;
            float *dst = y + (t * n_head + h) * ne0;
            const int64_t n_offset = mode == 0 ? 1 : n_dims / 2;
            const int64_t scale = mode == 0 ? 1 : 2;
            for (int64_t i0 = 0; i0 < n_dims; i0 += 2) {
                const int64_t ic = i0 / scale;
                const float c = cache[i0], s = cache[i0 + 1];
                const float x0 = src[ic], x1 = src[ic + n_offset];
                dst[ic] = std::fmaf(x0, c, -(x1 * s));
                dst[ic + n_offset] = std::fmaf(x0, s, x1 * c);
            }
            for (int64_t i0 = n_dims; i0 < ne0; i0++) dst[i0] = src[i0];
        }
    }
    return 0;
}

// crates/ggml/src/compute.rs:4265-4338 forward_set_rows, F32 rows -> F16 destination (round to
// nearest even), I64 row indices.  Returns -1 for an index outside [0, dst_rows).
int orc_set_rows_f16(const float *x, int64_t ne0, int64_t nrows, const int64_t *idx, uint16_t *dst, int64_t dst_rows) {
    for (int64_t r = 0; r < nrows; r++) {
        if (idx[r] < 0 || idx[r] >= dst_rows) return -1;
        uint16_t *d = dst + idx[r] * ne0;
        for (int64_t i = 0; i < ne0; i++) d[i] = orc_f32_to_f16(x[r * ne0 + i]);
    }
    return 0;
}

// crates/ggml/src/compute.rs:3842-3895 forward_get_rows: row ids[i] of a quantized / F16 / F32
// table to f32.  Returns -1 for an id outside the table or an unsupported type.
int orc_get_rows(int type, const void *table, int64_t ne0, int64_t table_rows, const int32_t *ids, int64_t n, float *y) {
    const size_t rs = type == ORC_F32 ? (size_t)ne0 * 4 : type == ORC_F16 ? (size_t)ne0 * 2 : orc_row_size(type, ne0);
    if (rs == 0) return -1;
    for (int64_t i = 0; i < n; i++) {
        if (ids[i] < 0 || ids[i] >= table_rows) return -1;
        const uint8_t *row = (const uint8_t *)table + (size_t)ids[i] * rs;
        float *out = y + i * ne0;
        if (type == ORC_F32) {
            std::memcpy(out, row, rs);
        } else if (type == ORC_F16) {
            for (int64_t j = 0; j < ne0; j++) out[j] = orc_f16_to_f32(((const uint16_t *)row)[j]);
        } else if (orc_dequantize_row(type, row, out, ne0) != 0) {
            return -1;
        }
    }
    return 0;
}

// crates/ggml/src/compute.rs:4208-4228 forward_argmax: ties resolve to the last occurrence
int32_t orc_argmax(const float *x, int64_t n) {
    float max = -std::numeric_limits<float>::infinity();
    int64_t idx = 0;
    for (int64_t i = 0; i < n; i++) {
        max = x[i] > max ? x[i] : max;
        if (max == x[i]) idx = i;
    }
    return (int32_t)idx;
}

// ---- Llama forward ------------------------------------------------------------------------------
// The node sequence of crates/llama/src/graph_arch.rs:106-248 build_llama_forward with the
// flash-attention branch of attn_kv_cached (:1173-1240), norm = rms_norm * weight (:1119-1122),
// FFN = down(silu(gate x) * (up x)) (:1128-1158), head over the gathered output rows
// (crates/llama/src/graph.rs:308-313).  No biases, no LoRA, one sequence.
struct OrcLlamaLayer {
    const void *wq, *wk, *wv, *wo, *gate, *up, *down;
    int32_t tq, tk, tv, to, tg, tu, td;
    const float *attn_norm, *ffn_norm;
    uint16_t *k_cache, *v_cache;   // [kv_size][n_head_kv * head_dim] F16
};
struct OrcLlamaModel {
    int32_t n_vocab, n_embd, n_head, n_head_kv, head_dim, n_ff, n_layer;
    int32_t rope_mode, n_ctx_orig, tok_type, out_type;
    float norm_eps, freq_base, freq_scale;
    const void *tok_embd;
    const float *out_norm;
    const void *output;
    OrcLlamaLayer *layers;
    int64_t kv_size;
};

// The reference interleaves a weight for the 8x8 kernels once, at load (crates/ggml/src/compute.rs:698-775).
// orc_mul_mat redoes it on every call, which is right for a checker and wrong for a stopwatch: with
// keep_repacked the forward pass keeps the interleaved copy of each weight it meets, keyed by address
// (only for callers whose weights stay put for the life of the process; orc_llama_drop_repacked forgets them).
static std::unordered_map<const void *, std::vector<uint8_t>> g_repacked;
void orc_llama_drop_repacked() { g_repacked.clear(); }
static int llama_mm(int type, int64_t N, int64_t K, int64_t M, const void *W, const float *X, float *out, int n_threads, int keep) {
    if (!keep || orc_pick_route(type, N, M) != ORC_ROUTE_REPACK) return orc_mul_mat(type, N, K, M, W, X, out, ORC_ROUTE_AUTO, n_threads);
    auto it = g_repacked.find(W);
    if (it == g_repacked.end()) {
        std::vector<uint8_t> rep(orc_row_size(type, K) * (size_t)N);
        if (orc_repack_8x8(type, W, N, K, rep.data()) != 0) return -1;
        it = g_repacked.emplace(W, std::move(rep)).first;
    }
    return orc_mul_mat_repacked(type, N, K, M, it->second.data(), X, out, n_threads);
}

// tokens / pos: [n_tok]; row_idx: [n_tok] cache cells to write; mask: F16 [n_tok][n_kv];
// out_ids: [n_out] token rows whose logits are wanted; logits: [n_out][n_vocab].
// Row-split tensor parallelism, restated on one host: attn_output and ffn_down are cut along K into tp slices on
// 256-element boundaries; slice r multiplies the matching columns of the activations (its own Q8 blocks: the cut
// is block-aligned, so they are the blocks the unsplit row would have), and the tp partial results are added in
// rank order, ((p0 + p1) + p2) + ..., each add rounded to f32.  Every other mat-mul is split by rows, which
// changes no output element.  partials, if given, receives the tp partial results [tp][M][N] before the sum.
static int llama_mm_ksplit(int type, int64_t N, int64_t K, int64_t M, const void *W, const float *X, float *out, int n_threads, int tp,
                           float *partials) {
    const size_t rb = orc_row_size(type, K);
    if (tp < 1 || K % tp != 0 || rb % (size_t)tp != 0 || (K / tp) % 256 != 0) return -1;
    const int64_t Ks = K / tp;
    const size_t srb = rb / (size_t)tp;
    std::vector<uint8_t> ws(srb * (size_t)N);
    std::vector<float> xs((size_t)M * Ks), part((size_t)M * N);
    for (int r = 0; r < tp; r++) {
        for (int64_t n = 0; n < N; n++) std::memcpy(ws.data() + (size_t)n * srb, (const uint8_t *)W + (size_t)n * rb + (size_t)r * srb, srb);
        for (int64_t i = 0; i < M; i++) std::memcpy(xs.data() + (size_t)i * Ks, X + (size_t)i * K + (size_t)r * Ks, (size_t)Ks * 4);
        if (orc_mul_mat(type, N, Ks, M, ws.data(), xs.data(), part.data(), ORC_ROUTE_AUTO, n_threads) < 0) return -1;
        if (partials) std::memcpy(partials + (size_t)r * M * N, part.data(), (size_t)M * N * 4);
        if (r == 0) std::memcpy(out, part.data(), (size_t)M * N * 4);
        else orc_add(out, part.data(), out, N, M, N, M);
    }
    return 1;
}

static int llama_forward_impl(const OrcLlamaModel *m, const int32_t *tokens, const int32_t *pos, int64_t n_tok, int64_t n_kv,
                              const uint16_t *mask, const int64_t *row_idx, const int32_t *out_ids, int64_t n_out, float *logits,
                              int n_threads, int wide_silu, int keep_repacked, int tp, float *attn_partials0, float *ffn_partials0);

int orc_llama_forward(const OrcLlamaModel *m, const int32_t *tokens, const int32_t *pos, int64_t n_tok, int64_t n_kv,
                      const uint16_t *mask, const int64_t *row_idx, const int32_t *out_ids, int64_t n_out, float *logits,
                      int n_threads, int wide_silu, int keep_repacked) {
    return llama_forward_impl(m, tokens, pos, n_tok, n_kv, mask, row_idx, out_ids, n_out, logits, n_threads, wide_silu, keep_repacked, 1,
                              nullptr, nullptr);
}

// The same forward pass as a group of tp tensor-parallel ranks computes it (see llama_mm_ksplit).  attn_partials0 /
// ffn_partials0, if given, receive layer 0's per-rank partial results of attn_output / ffn_down, [tp][n_tok][n_embd].
int orc_llama_forward_tp(const OrcLlamaModel *m, const int32_t *tokens, const int32_t *pos, int64_t n_tok, int64_t n_kv,
                         const uint16_t *mask, const int64_t *row_idx, const int32_t *out_ids, int64_t n_out, float *logits,
                         int n_threads, int wide_silu, int tp, float *attn_partials0, float *ffn_partials0) {
    if (tp < 1 || m->n_head % tp || m->n_head_kv % tp || m->n_ff % tp) return -7;
    return llama_forward_impl(m, tokens, pos, n_tok, n_kv, mask, row_idx, out_ids, n_out, logits, n_threads, wide_silu, 0, tp,
                              attn_partials0, ffn_partials0);
}

static int llama_forward_impl(const OrcLlamaModel *m, const int32_t *tokens, const int32_t *pos, int64_t n_tok, int64_t n_kv,
                              const uint16_t *mask, const int64_t *row_idx, const int32_t *out_ids, int64_t n_out, float *logits,
                              int n_threads, int wide_silu, int keep_repacked, int tp, float *attn_partials0, float *ffn_partials0) {
    const int64_t E = m->n_embd, HD = m->head_dim, H = m->n_head, HK = m->n_head_kv, FF = m->n_ff, T = n_tok;
    const int64_t EK = HK * HD;
    std::vector<float> inp(T * E), cur(T * E), q(T * H * HD), k(T * EK), v(T * EK), qr(T * H * HD), kr(T * EK);
    std::vector<float> att(T * H * HD), proj(T * E), ffn_inp(T * E), g(T * FF), u(T * FF);
    if (orc_get_rows(m->tok_type, m->tok_embd, E, m->n_vocab, tokens, T, inp.data()) != 0) return -1;
    const float kq_scale = 1.0f / std::sqrt((float)HD);
    for (int il = 0; il < m->n_layer; il++) {
        const OrcLlamaLayer &L = m->layers[il];
        orc_rms_norm(inp.data(), cur.data(), E, T, m->norm_eps);
        orc_mul(cur.data(), L.attn_norm, cur.data(), E, T, E, 1);
        if (llama_mm(L.tq, H * HD, E, T, L.wq, cur.data(), q.data(), n_threads, keep_repacked) < 0) return -2;
        if (llama_mm(L.tk, EK, E, T, L.wk, cur.data(), k.data(), n_threads, keep_repacked) < 0) return -2;
        if (llama_mm(L.tv, EK, E, T, L.wv, cur.data(), v.data(), n_threads, keep_repacked) < 0) return -2;
        if (orc_rope(q.data(), qr.data(), HD, H, T, pos, nullptr, (int)HD, m->rope_mode, m->n_ctx_orig, m->freq_base,
                     m->freq_scale, 0.0f, 1.0f, 32.0f, 1.0f) != 0) return -3;
        if (orc_rope(k.data(), kr.data(), HD, HK, T, pos, nullptr, (int)HD, m->rope_mode, m->n_ctx_orig, m->freq_base,
                     m->freq_scale, 0.0f, 1.0f, 32.0f, 1.0f) != 0) return -3;
        if (orc_set_rows_f16(kr.data(), EK, T, row_idx, L.k_cache, m->kv_size) != 0) return -4;
        if (orc_set_rows_f16(v.data(), EK, T, row_idx, L.v_cache, m->kv_size) != 0) return -4;
        OrcFlashArgs fa;
        std::memset(&fa, 0, sizeof(fa));
        fa.dk = HD; fa.dv = HD; fa.T = T; fa.H = H; fa.H_kv = HK; fa.n_kv = n_kv;
        fa.q = qr.data(); fa.q_nb1 = H * HD * 4; fa.q_nb2 = HD * 4;
        fa.k = L.k_cache; fa.k_nb1 = EK * 2; fa.k_nb2 = HD * 2;
        fa.v = L.v_cache; fa.v_nb1 = EK * 2; fa.v_nb2 = HD * 2;
        fa.mask = mask; fa.mask_nb1 = n_kv * 2;
        fa.scale = kq_scale;
        fa.dst = att.data();
        fa.mode = 0; fa.n_chunks = n_threads; fa.n_threads = n_threads;
        if (orc_flash_attn_ext(&fa) <= 0) return -5;
        if (tp > 1) {
            if (llama_mm_ksplit(L.to, E, H * HD, T, L.wo, att.data(), proj.data(), n_threads, tp, il == 0 ? attn_partials0 : nullptr) < 0) return -2;
        } else if (llama_mm(L.to, E, H * HD, T, L.wo, att.data(), proj.data(), n_threads, keep_repacked) < 0) return -2;
        orc_add(proj.data(), inp.data(), ffn_inp.data(), E, T, E, T);
        orc_rms_norm(ffn_inp.data(), cur.data(), E, T, m->norm_eps);
        orc_mul(cur.data(), L.ffn_norm, cur.data(), E, T, E, 1);
        if (llama_mm(L.tg, FF, E, T, L.gate, cur.data(), g.data(), n_threads, keep_repacked) < 0) return -2;
        if (llama_mm(L.tu, FF, E, T, L.up, cur.data(), u.data(), n_threads, keep_repacked) < 0) return -2;
        orc_silu(g.data(), g.data(), FF, T, wide_silu);
        orc_mul(g.data(), u.data(), g.data(), FF, T, FF, T);
        if (tp > 1) {
            if (llama_mm_ksplit(L.td, E, FF, T, L.down, g.data(), proj.data(), n_threads, tp, il == 0 ? ffn_partials0 : nullptr) < 0) return -2;
        } else if (llama_mm(L.td, E, FF, T, L.down, g.data(), proj.data(), n_threads, keep_repacked) < 0) return -2;
        orc_add(proj.data(), ffn_inp.data(), inp.data(), E, T, E, T);
    }
    orc_rms_norm(inp.data(), cur.data(), E, T, m->norm_eps);
    orc_mul(cur.data(), m->out_norm, cur.data(), E, T, E, 1);
    std::vector<float> rows(n_out * E);
    for (int64_t i = 0; i < n_out; i++) {
        if (out_ids[i] < 0 || out_ids[i] >= T) return -6;
        std::memcpy(rows.data() + i * E, cur.data() + (int64_t)out_ids[i] * E, E * 4);
    }
    if (llama_mm(m->out_type, m->n_vocab, E, n_out, m->output, rows.data(), logits, n_threads, keep_repacked) < 0) return -2;
    return 0;
}

}  // extern "C"
