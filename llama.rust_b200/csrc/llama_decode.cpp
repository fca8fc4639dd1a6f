// A Llama decode driver over the ggml backend plug-in (include/llama_b200.h).
//
// The reference's DecodeContext (crates/llama/src/context.rs) owns the weights, the KV cache and the
// per-step input tensors, builds the forward graph and hands it to a backend.  This file does the same
// for the llama architecture with this library's own backend, and it talks to that backend only
// through the vtables a foreign host would use: get_alloc_size / alloc_buffer / set_tensor /
// graph_compute / get_tensor_async.  The nodes are emitted in the order the reference's graph gets them
// (depth-first from the roots it expands: each layer's input, the two cache writes, the logits).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "ggml_b200_backend.h"
#include "llama_b200.h"
#include "tp.h"

using namespace b200;

namespace {

constexpr size_t ALIGN = 256;
constexpr int64_t KV_PAD = 256;   // crates/llama/src/kv_cache.rs:1887-1917: n_kv is padded to 256 cells

size_t type_size(int type) {
    switch (type) {
        case B200_TYPE_F32: case B200_TYPE_I32: return 4;
        case B200_TYPE_F16: return 2;
        case B200_TYPE_I64: return 8;
        default: return 0;
    }
}
size_t quant_row_bytes(int type, int64_t ne0) { return (size_t)(ne0 / GROUP_K) * group_src_bytes(type); }

struct Weight {
    ggml_tensor t;
    ggml_backend_buffer_t buf = nullptr;
};

struct Graph {
    std::deque<ggml_tensor> tensors;      // stable addresses
    std::vector<ggml_tensor *> nodes;
    ggml_tensor *tokens = nullptr, *pos = nullptr, *mask = nullptr, *row_idx = nullptr, *out_ids = nullptr;
    ggml_tensor *logits = nullptr, *argmax = nullptr;
    size_t bytes = 0;                     // compute-buffer bytes the graph spans
};

}  // namespace

struct b200_llama {
    b200_llama_hparams hp;
    int32_t n_ctx = 0, n_batch = 0;
    ggml_backend_dev_t dev = nullptr;
    ggml_backend_t backend = nullptr;
    ggml_backend_buffer_type_t buft = nullptr;
    void *stream = nullptr;
    std::map<std::string, std::unique_ptr<Weight>> weights;
    ggml_backend_buffer_t kv_buf = nullptr, compute_buf = nullptr;
    std::vector<ggml_tensor> k_l, v_l;    // [n_embd_k_gqa, n_ctx] F16 per layer
    std::vector<int32_t> cell_pos;        // position held by each cache cell, -1 = empty
    std::vector<int32_t> cell_seq;        // the sequence the cell belongs to
    int32_t used = 0;
    std::map<std::pair<int64_t, int64_t>, std::unique_ptr<Graph>> graphs;   // by (n_tokens, n_kv)
    Graph *last = nullptr;
    std::vector<uint16_t> mask_host;
    std::vector<int64_t> idx_host;
    // tensor parallel: this rank holds n_head / tp_size heads, n_head_kv / tp_size cache heads, the matching
    // rows / columns of every matrix (tp.cpp) and 1 / tp_size of the vocabulary rows
    int32_t tp_rank = 0, tp_size = 1;
    TpGroup *tp = nullptr;
    std::vector<uint8_t> shard_tmp;
};

namespace {

void init_tensor(ggml_tensor *t, int type, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1, int64_t ne3 = 1) {
    memset(t, 0, sizeof(*t));
    t->type = type;
    t->ne[0] = ne0; t->ne[1] = ne1; t->ne[2] = ne2; t->ne[3] = ne3;
    const size_t row = is_quant_type(type) ? quant_row_bytes(type, ne0) : type_size(type) * (size_t)ne0;
    t->nb[0] = is_quant_type(type) ? (size_t)group_src_bytes(type) / (type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K ? 1 : 8) : type_size(type);
    t->nb[1] = row;
    t->nb[2] = t->nb[1] * (size_t)ne1;
    t->nb[3] = t->nb[2] * (size_t)ne2;
}

// One pass over the compute buffer: tensors are placed back to back; a layer's intermediates are
// placed again over the previous layer's (everything runs in order on one stream).
struct Builder {
    b200_llama *c;
    Graph *g;
    uint8_t *base;
    size_t off = 0, high = 0;

    ggml_tensor *fresh(int type, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1, int64_t ne3 = 1) {
        g->tensors.emplace_back();
        ggml_tensor *t = &g->tensors.back();
        init_tensor(t, type, ne0, ne1, ne2, ne3);
        return t;
    }
    ggml_tensor *alloc(int type, int64_t ne0, int64_t ne1 = 1, int64_t ne2 = 1, const char *name = "") {
        ggml_tensor *t = fresh(type, ne0, ne1, ne2);
        off = (off + ALIGN - 1) / ALIGN * ALIGN;
        t->data = base ? base + off : nullptr;
        t->buffer = c->compute_buf;
        off += t->nb[3];
        high = std::max(high, off);
        snprintf(t->name, sizeof(t->name), "%s", name);
        return t;
    }
    ggml_tensor *op(ggml_tensor *t, int code, ggml_tensor *a, ggml_tensor *b = nullptr, ggml_tensor *c2 = nullptr, ggml_tensor *d = nullptr) {
        t->op = code;
        t->src[0] = a; t->src[1] = b; t->src[2] = c2; t->src[3] = d;
        g->nodes.push_back(t);
        return t;
    }
    // an alias of src's bytes with its own shape and strides (RESHAPE / VIEW / PERMUTE nodes)
    ggml_tensor *alias(int code, ggml_tensor *src, size_t offset, const int64_t ne[4], const size_t nb[4], const char *name = "") {
        ggml_tensor *t = fresh(src->type, 1);
        for (int i = 0; i < 4; i++) { t->ne[i] = ne[i]; t->nb[i] = nb[i]; }
        t->view_src = src->view_src ? src->view_src : src;
        t->view_offs = src->view_offs + offset;
        t->data = src->data ? (uint8_t *)src->data + offset : nullptr;
        t->buffer = src->buffer;
        snprintf(t->name, sizeof(t->name), "%s", name);
        return op(t, code, src);
    }
    ggml_tensor *reshape_3d(ggml_tensor *a, int64_t ne0, int64_t ne1, int64_t ne2) {
        const int64_t ne[4] = {ne0, ne1, ne2, 1};
        const size_t es = a->nb[0];
        const size_t nb[4] = {es, es * ne0, es * ne0 * ne1, es * ne0 * ne1 * ne2};
        return alias(GGML_OP_RESHAPE, a, 0, ne, nb);
    }
    ggml_tensor *reshape_2d(ggml_tensor *a, int64_t ne0, int64_t ne1) { return reshape_3d(a, ne0, ne1, 1); }
    ggml_tensor *view_2d(ggml_tensor *a, int64_t ne0, int64_t ne1, size_t nb1, size_t offset) {
        const int64_t ne[4] = {ne0, ne1, 1, 1};
        const size_t nb[4] = {a->nb[0], nb1, nb1 * ne1, nb1 * ne1};
        return alias(GGML_OP_VIEW, a, offset, ne, nb);
    }
    ggml_tensor *view_3d(ggml_tensor *a, int64_t ne0, int64_t ne1, int64_t ne2, size_t nb1, size_t nb2, size_t offset) {
        const int64_t ne[4] = {ne0, ne1, ne2, 1};
        const size_t nb[4] = {a->nb[0], nb1, nb2, nb2 * ne2};
        return alias(GGML_OP_VIEW, a, offset, ne, nb);
    }
    // permute(a, 0, 2, 1, 3): swap dims 1 and 2
    ggml_tensor *permute_0213(ggml_tensor *a) {
        const int64_t ne[4] = {a->ne[0], a->ne[2], a->ne[1], a->ne[3]};
        const size_t nb[4] = {a->nb[0], a->nb[2], a->nb[1], a->nb[3]};
        return alias(GGML_OP_PERMUTE, a, 0, ne, nb);
    }
    ggml_tensor *mul_mat(ggml_tensor *w, ggml_tensor *x, const char *name = "") {
        return op(alloc(B200_TYPE_F32, w->ne[1], x->ne[1], 1, name), GGML_OP_MUL_MAT, w, x);
    }
    ggml_tensor *binary(int code, ggml_tensor *a, ggml_tensor *b, const char *name = "") {
        return op(alloc(B200_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], name), code, a, b);
    }
    // a new tensor over the bytes of `slot` (the residual stream alternates between two slots)
    ggml_tensor *over(const ggml_tensor *slot, const char *name) {
        ggml_tensor *t = fresh(slot->type, slot->ne[0], slot->ne[1], slot->ne[2]);
        t->data = slot->data;
        t->buffer = slot->buffer;
        snprintf(t->name, sizeof(t->name), "%s", name);
        return t;
    }
    ggml_tensor *rms_norm(ggml_tensor *a, float eps) {
        ggml_tensor *t = op(alloc(B200_TYPE_F32, a->ne[0], a->ne[1], a->ne[2]), GGML_OP_RMS_NORM, a);
        memcpy(&t->op_params[0], &eps, 4);
        return t;
    }
    // crates/llama/src/graph_arch.rs:1119-1122 build_norm_rms
    ggml_tensor *norm(ggml_tensor *a, ggml_tensor *w, float eps, const char *name) { return binary(GGML_OP_MUL, rms_norm(a, eps), w, name); }
    ggml_tensor *silu(ggml_tensor *a) {
        ggml_tensor *t = op(alloc(B200_TYPE_F32, a->ne[0], a->ne[1], a->ne[2]), GGML_OP_UNARY, a);
        t->op_params[0] = GGML_UNARY_OP_SILU;
        return t;
    }
    // crates/ggml/src/ops.rs rope_ext: op_params = [n_past, n_dims, mode, n_ctx, n_ctx_orig, freq_base, freq_scale,
    // ext_factor, attn_factor, beta_fast, beta_slow, sections[4], n_offs]
    ggml_tensor *rope(ggml_tensor *a, ggml_tensor *pos, const char *name) {
        const b200_llama_hparams &hp = c->hp;
        ggml_tensor *t = op(alloc(B200_TYPE_F32, a->ne[0], a->ne[1], a->ne[2], name), GGML_OP_ROPE, a, pos);
        const float f[6] = {hp.rope_freq_base, hp.rope_freq_scale, 0.0f, 1.0f, 32.0f, 1.0f};
        t->op_params[1] = hp.n_embd_head;
        t->op_params[2] = hp.rope_mode;
        t->op_params[4] = hp.n_ctx_train;
        memcpy(&t->op_params[5], f, sizeof(f));
        return t;
    }
    // set_rows(cache, rows, idx): the result aliases the cache tensor
    ggml_tensor *set_rows(ggml_tensor *cache, ggml_tensor *rows, ggml_tensor *idx) {
        ggml_tensor *t = fresh(cache->type, 1);
        for (int i = 0; i < 4; i++) { t->ne[i] = cache->ne[i]; t->nb[i] = cache->nb[i]; }
        t->view_src = cache;
        t->data = cache->data;
        t->buffer = cache->buffer;
        return op(t, GGML_OP_SET_ROWS, rows, idx);
    }
    // the sum of a over the ranks of the tensor-parallel group, in place: the node aliases a
    ggml_tensor *tp_all_reduce(ggml_tensor *a, const char *name) {
        ggml_tensor *t = fresh(a->type, a->ne[0], a->ne[1], a->ne[2]);
        t->data = a->data;
        t->buffer = a->buffer;
        t->view_src = a->view_src ? a->view_src : a;
        t->view_offs = a->view_offs;
        snprintf(t->name, sizeof(t->name), "%s", name);
        return op(t, B200_OP_TP_ALL_REDUCE, a);
    }
    ggml_tensor *get_rows(ggml_tensor *table, ggml_tensor *ids, const char *name = "") {
        return op(alloc(B200_TYPE_F32, table->ne[0], ids->ne[0], 1, name), GGML_OP_GET_ROWS, table, ids);
    }
};

ggml_tensor *weight(b200_llama *c, const std::string &name) {
    auto it = c->weights.find(name);
    return it == c->weights.end() ? nullptr : &it->second->t;
}

// crates/llama/src/graph_arch.rs:106-248 with attn_kv_cached's flash-attention branch (:1173-1240) and
// build_ffn_silu_par (:1128-1158).  base == nullptr only measures.
int build_graph(b200_llama *c, Graph *g, uint8_t *base, int64_t n, int64_t n_kv, int64_t n_out) {
    const b200_llama_hparams &hp = c->hp;
    const int64_t E = hp.n_embd, HD = hp.n_embd_head, H = hp.n_head / c->tp_size, HK = hp.n_head_kv / c->tp_size, EK = HK * HD;
    const bool tp = c->tp_size > 1;
    Builder b{c, g, base};
    g->tokens = b.alloc(B200_TYPE_I32, n, 1, 1, "inp_tokens");
    g->pos = b.alloc(B200_TYPE_I32, n, 1, 1, "inp_pos");
    g->mask = b.alloc(B200_TYPE_F16, n_kv, n, 1, "kq_mask");
    g->row_idx = b.alloc(B200_TYPE_I64, n, 1, 1, "kv_idxs");
    g->out_ids = b.alloc(B200_TYPE_I32, n_out, 1, 1, "inp_out_ids");
    ggml_tensor *resid[2] = {b.alloc(B200_TYPE_F32, E, n, 1, "resid_a"), b.alloc(B200_TYPE_F32, E, n, 1, "resid_b")};

    ggml_tensor *tok_embd = weight(c, "token_embd.weight");
    B200_REQUIRE(tok_embd != nullptr, "llama: token_embd.weight has not been set");
    ggml_tensor *inp = b.op(b.over(resid[0], "inp_embd"), GGML_OP_GET_ROWS, tok_embd, g->tokens);
    const size_t layer_base = b.off;
    const float kq_scale = 1.0f / sqrtf((float)HD);

    for (int il = 0; il < hp.n_layer; il++) {
        b.off = layer_base;
        const std::string p = "blk." + std::to_string(il) + ".";
        ggml_tensor *wq = weight(c, p + "attn_q.weight"), *wk = weight(c, p + "attn_k.weight"), *wv = weight(c, p + "attn_v.weight");
        ggml_tensor *wo = weight(c, p + "attn_output.weight"), *an = weight(c, p + "attn_norm.weight"), *fn = weight(c, p + "ffn_norm.weight");
        ggml_tensor *wg = weight(c, p + "ffn_gate.weight"), *wu = weight(c, p + "ffn_up.weight"), *wd = weight(c, p + "ffn_down.weight");
        B200_REQUIRE(wq && wk && wv && wo && an && fn && wg && wu && wd, "llama: layer %d is missing a tensor", il);

        ggml_tensor *cur = b.norm(inp, an, hp.norm_rms_eps, "attn_norm");
        // root 1: the K cache write
        ggml_tensor *k = b.reshape_3d(b.mul_mat(wk, cur, "Kcur"), HD, HK, n);
        k = b.rope(k, g->pos, "Kcur_rope");
        ggml_tensor *k_rows = b.view_2d(k, EK, n, k->nb[2], 0);
        b.set_rows(&c->k_l[il], k_rows, g->row_idx);
        // root 2: the V cache write
        ggml_tensor *v = b.reshape_3d(b.mul_mat(wv, cur, "Vcur"), HD, HK, n);
        ggml_tensor *v_rows = b.view_2d(v, EK, n, v->nb[2], 0);
        b.set_rows(&c->v_l[il], v_rows, g->row_idx);
        // root 3: the layer output, reached through the attention
        ggml_tensor *q = b.reshape_3d(b.mul_mat(wq, cur, "Qcur"), HD, H, n);
        q = b.rope(q, g->pos, "Qcur_rope");
        ggml_tensor *q_fa = b.permute_0213(q);
        // KvCache::get_k / get_v: [head, n_head_kv, n_kv] views of the layer's cache, then [head, n_kv, n_head_kv]
        ggml_tensor *k_fa = b.permute_0213(b.view_3d(&c->k_l[il], HD, HK, n_kv, HD * 2, EK * 2, 0));
        ggml_tensor *v_fa = b.permute_0213(b.view_3d(&c->v_l[il], HD, HK, n_kv, HD * 2, EK * 2, 0));
        ggml_tensor *fa = b.op(b.alloc(B200_TYPE_F32, HD, H, n, "kqv_out"), GGML_OP_FLASH_ATTN_EXT, q_fa, k_fa, v_fa, g->mask);
        memcpy(&fa->op_params[0], &kq_scale, 4);
        ggml_tensor *attn = b.mul_mat(wo, b.reshape_2d(fa, HD * H, n), "attn_out");
        if (tp) attn = b.tp_all_reduce(attn, "attn_out_sum");   // attn holds the partial sums over this rank's heads
        ggml_tensor *ffn_inp = b.binary(GGML_OP_ADD, attn, inp, "ffn_inp");
        cur = b.norm(ffn_inp, fn, hp.norm_rms_eps, "ffn_norm");
        ggml_tensor *gate = b.silu(b.mul_mat(wg, cur, "ffn_gate"));
        ggml_tensor *up = b.mul_mat(wu, cur, "ffn_up");
        ggml_tensor *down = b.mul_mat(wd, b.binary(GGML_OP_MUL, gate, up, "ffn_gate_par"), "ffn_out");
        if (tp) down = b.tp_all_reduce(down, "ffn_out_sum");   // down holds the partial sums over this rank's FFN rows
        inp = b.op(b.over(resid[(il + 1) & 1], "l_out"), GGML_OP_ADD, down, ffn_inp);
    }
    b.off = layer_base;
    ggml_tensor *on = weight(c, "output_norm.weight");
    ggml_tensor *ow = weight(c, "output.weight");
    if (!ow) ow = tok_embd;   // tied embeddings
    B200_REQUIRE(on != nullptr, "llama: output_norm.weight has not been set");
    ggml_tensor *cur = b.norm(inp, on, hp.norm_rms_eps, "result_norm");
    cur = b.get_rows(cur, g->out_ids, "result_norm_rows");   // crates/llama/src/graph.rs:308-313 out_rows
    g->logits = b.mul_mat(ow, cur, "result_output");
    if (tp && ow != tok_embd) {   // this rank's vocabulary rows: gather the full row on every rank
        ggml_tensor *staging = b.alloc(B200_TYPE_F32, ow->ne[1] * c->tp_size, n_out, 1, "result_output_staging");
        g->logits = b.op(b.alloc(B200_TYPE_F32, ow->ne[1] * c->tp_size, n_out, 1, "result_output_all"), B200_OP_TP_ALL_GATHER, g->logits, staging);
    }
    g->argmax = b.op(b.alloc(B200_TYPE_I32, n_out, 1, 1, "argmax"), GGML_OP_ARGMAX, g->logits);
    g->bytes = b.high;
    return B200_STATUS_SUCCESS;
}

int64_t n_kv_for(const b200_llama *c, int32_t used) {
    // min(size, max(256, pad256(highest used cell + 1))): crates/llama/src/kv_cache.rs:1887-1917
    const int64_t padded = (used + KV_PAD - 1) / KV_PAD * KV_PAD;
    return std::min<int64_t>(c->n_ctx, std::max<int64_t>(KV_PAD, padded));
}

void set_input(ggml_tensor *t, const void *data, size_t bytes) { t->buffer->iface.set_tensor(t->buffer, t, data, 0, bytes); }
// the per-step inputs: ordered on the backend's stream ahead of the step's graph, no wait per copy
void set_input_async(ggml_backend_t be, ggml_tensor *t, const void *data, size_t bytes) {
    if (be->iface.set_tensor_async) be->iface.set_tensor_async(be, t, data, 0, bytes);
    else set_input(t, data, bytes);
}

// graph_compute over the first `total` nodes: the whole step is one node list, the collectives of a tensor-parallel
// group are nodes of it (B200_OP_TP_*), so the backend can capture and replay the step as one CUDA graph
int run_graph(b200_llama *c, Graph *g, int total) {
    ggml_cgraph cg;
    memset(&cg, 0, sizeof(cg));
    cg.size = cg.n_nodes = total;
    cg.nodes = g->nodes.data();
    return c->backend->iface.graph_compute(c->backend, &cg);
}

}  // namespace

extern "C" {

int b200_llama_new(const b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, b200_llama **out) {
    return b200_llama_new_tp(hp, device, n_ctx, n_batch, cpu_threads, 0, 1, nullptr, out);
}

static int llama_new_impl(const b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                          int32_t tp_size, const void *id128, b200_tp_hook_fn hook, void *hook_user, b200_llama **out);

int b200_llama_new_tp(const b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                      int32_t tp_size, const void *id128, b200_llama **out) {
    return llama_new_impl(hp, device, n_ctx, n_batch, cpu_threads, tp_rank, tp_size, id128, nullptr, nullptr, out);
}

int b200_llama_new_tp_hook(const b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                           int32_t tp_size, b200_tp_hook_fn hook, void *user, b200_llama **out) {
    B200_REQUIRE(hook != nullptr && tp_size >= 2, "llama_new_tp_hook: needs a hook and at least two ranks");
    return llama_new_impl(hp, device, n_ctx, n_batch, cpu_threads, tp_rank, tp_size, nullptr, hook, user, out);
}

int b200_llama_tp_exchange_kind(const b200_llama *c) {
    if (!c || !c->tp || c->tp->hook) return -1;
    return c->tp->ll_ready ? 1 : 0;
}

static int llama_new_impl(const b200_llama_hparams *hp, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                          int32_t tp_size, const void *id128, b200_tp_hook_fn hook, void *hook_user, b200_llama **out) {
    B200_REQUIRE(hp != nullptr && out != nullptr, "llama_new: null argument");
    *out = nullptr;
    B200_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "llama_new: rank %d of %d", tp_rank, tp_size);
    B200_REQUIRE(tp_size == 1 || id128 != nullptr || hook != nullptr, "llama_new: a tensor-parallel group needs the shared id");
    B200_REQUIRE(hp->n_head % tp_size == 0 && hp->n_head_kv % tp_size == 0, "llama_new: %d / %d heads do not split %d ways", hp->n_head,
                 hp->n_head_kv, tp_size);
    B200_REQUIRE(hp->n_vocab > 0 && hp->n_embd > 0 && hp->n_head > 0 && hp->n_head_kv > 0 && hp->n_layer > 0 && hp->n_ff > 0,
                 "llama_new: non-positive model dimension");
    B200_REQUIRE(hp->n_head % hp->n_head_kv == 0, "llama_new: n_head %d is not a multiple of n_head_kv %d", hp->n_head, hp->n_head_kv);
    B200_REQUIRE(hp->n_embd_head == 64 || hp->n_embd_head == 128, "llama_new: head size %d is not 64 or 128", hp->n_embd_head);
    B200_REQUIRE(hp->n_embd % GROUP_K == 0 && hp->n_ff % GROUP_K == 0 && (hp->n_head * hp->n_embd_head) % GROUP_K == 0,
                 "llama_new: n_embd, n_ff and n_head * head size must be multiples of 256");
    B200_REQUIRE(hp->rope_mode == 0 || hp->rope_mode == 2, "llama_new: rope mode %d is neither NORMAL (0) nor NEOX (2)", hp->rope_mode);
    B200_REQUIRE((hp->n_head / tp_size * hp->n_embd_head) % GROUP_K == 0 && (hp->n_ff / tp_size) % GROUP_K == 0 && hp->n_ff % tp_size == 0,
                 "llama_new: a rank's share of the heads and of n_ff must be multiples of 256 elements");
    B200_REQUIRE(n_ctx > 0 && n_ctx % KV_PAD == 0, "llama_new: n_ctx %d must be a positive multiple of 256", n_ctx);
    B200_REQUIRE(n_batch > 0 && n_batch <= n_ctx, "llama_new: n_batch %d out of (0, n_ctx]", n_batch);
    ggml_backend_reg_t reg = ggml_backend_init();
    B200_REQUIRE(reg != nullptr && reg->api_version == GGML_BACKEND_API_VERSION, "llama_new: backend registry unavailable");
    ggml_backend_dev_t dev = reg->iface.get_device(reg, (size_t)device);
    B200_REQUIRE(dev != nullptr, "llama_new: no usable device %d", device);
    std::unique_ptr<b200_llama> c(new b200_llama());
    c->hp = *hp;
    c->n_ctx = n_ctx;
    c->n_batch = n_batch;
    c->dev = dev;
    c->tp_rank = tp_rank;
    c->tp_size = tp_size;
    const std::string params = "cpu_threads=" + std::to_string(cpu_threads > 0 ? cpu_threads : 8);
    c->backend = dev->iface.init_backend(dev, params.c_str());
    if (!c->backend) return B200_STATUS_BACKEND_ERROR;
    c->buft = dev->iface.get_buffer_type(dev);
    typedef void *(*get_stream_fn)(ggml_backend_t);
    get_stream_fn get_stream = (get_stream_fn)reg->iface.get_proc_address(reg, "b200_backend_get_stream");
    c->stream = get_stream ? get_stream(c->backend) : nullptr;

    // KV cache: per layer K and V, [n_embd_k_gqa, n_ctx] F16, zero-filled
    const int64_t EK = (int64_t)hp->n_head_kv / tp_size * hp->n_embd_head;
    const size_t per = ((size_t)EK * 2 * n_ctx + ALIGN - 1) / ALIGN * ALIGN;
    c->kv_buf = c->buft->iface.alloc_buffer(c->buft, per * 2 * hp->n_layer);
    if (!c->kv_buf) { b200_llama_free(c.release()); return B200_STATUS_ALLOC_FAILED; }
    c->kv_buf->iface.clear(c->kv_buf, 0);
    c->k_l.resize(hp->n_layer);
    c->v_l.resize(hp->n_layer);
    uint8_t *kvb = (uint8_t *)c->kv_buf->iface.get_base(c->kv_buf);
    for (int il = 0; il < hp->n_layer; il++) {
        for (int which = 0; which < 2; which++) {
            ggml_tensor *t = which ? &c->v_l[il] : &c->k_l[il];
            init_tensor(t, B200_TYPE_F16, EK, n_ctx);
            t->buffer = c->kv_buf;
            t->data = kvb + per * (2 * il + which);
            snprintf(t->name, sizeof(t->name), "cache_%c_l%d", which ? 'v' : 'k', il);
        }
    }
    c->cell_pos.assign(n_ctx, -1);
    c->cell_seq.assign(n_ctx, -1);
    if (tp_size > 1) {
        int rc = tp_group_create(tp_rank, tp_size, device, id128, hook, hook_user, &c->tp);
        if (rc != B200_STATUS_SUCCESS) { b200_llama_free(c.release()); return rc; }
        typedef void (*set_tp_fn)(ggml_backend_t, void *);
        set_tp_fn set_tp = (set_tp_fn)reg->iface.get_proc_address(reg, "b200_backend_set_tp");
        if (!set_tp) { b200_llama_free(c.release()); B200_REQUIRE(false, "llama_new: the backend has no tensor-parallel entry"); }
        set_tp(c->backend, c->tp);
    }
    *out = c.release();
    return B200_STATUS_SUCCESS;
}

void b200_llama_free(b200_llama *c) {
    if (!c) return;
    if (c->backend) c->backend->iface.synchronize(c->backend);
    c->graphs.clear();
    if (c->compute_buf) c->compute_buf->iface.free_buffer(c->compute_buf);
    if (c->kv_buf) c->kv_buf->iface.free_buffer(c->kv_buf);
    for (auto &kv : c->weights)
        if (kv.second->buf) kv.second->buf->iface.free_buffer(kv.second->buf);
    if (c->backend) c->backend->iface.free(c->backend);
    if (c->tp) tp_group_destroy(c->tp);
    delete c;
}

static int set_tensor_impl(b200_llama *c, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes, bool whole);

int b200_llama_set_tensor(b200_llama *c, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes) {
    return set_tensor_impl(c, name, type, ne0, ne1, data, nbytes, true);
}
int b200_llama_set_tensor_shard(b200_llama *c, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes) {
    return set_tensor_impl(c, name, type, ne0, ne1, data, nbytes, false);
}

static int set_tensor_impl(b200_llama *c, const char *name, int type, int64_t ne0, int64_t ne1, const void *data, size_t nbytes, bool whole) {
    B200_REQUIRE(c != nullptr && name != nullptr && data != nullptr, "llama_set_tensor: null argument");
    B200_REQUIRE(ne0 > 0 && ne1 > 0, "llama_set_tensor: %s has an empty shape", name);
    const bool quant = is_quant_type(type);
    B200_REQUIRE(quant || type == B200_TYPE_F32 || type == B200_TYPE_F16, "llama_set_tensor: %s: type %d is not supported", name, type);
    B200_REQUIRE(!quant || ne0 % GROUP_K == 0, "llama_set_tensor: %s: row length %lld is not a multiple of 256", name, (long long)ne0);
    std::unique_ptr<Weight> w(new Weight());
    init_tensor(&w->t, type, ne0, ne1);
    B200_REQUIRE(nbytes == w->t.nb[2], "llama_set_tensor: %s: %zu bytes given, %zu expected", name, nbytes, w->t.nb[2]);
    if (c->tp_size > 1 && whole) {   // keep this rank's shard of the whole tensor
        int32_t split = 0;
        int64_t l0 = 0, l1 = 0;
        int rc = b200_tp_shard_shape(name, type, ne0, ne1, c->tp_size, &split, &l0, &l1);
        if (rc != B200_STATUS_SUCCESS) return rc;
        if (split != 0) {
            init_tensor(&w->t, type, l0, l1);
            c->shard_tmp.resize(w->t.nb[2]);
            rc = b200_tp_shard_tensor(name, type, ne0, ne1, data, c->tp_rank, c->tp_size, c->shard_tmp.data(), c->shard_tmp.size());
            if (rc != B200_STATUS_SUCCESS) return rc;
            data = c->shard_tmp.data();
            nbytes = c->shard_tmp.size();
        }
    }
    snprintf(w->t.name, sizeof(w->t.name), "%s", name);
    w->buf = c->buft->iface.alloc_buffer(c->buft, c->buft->iface.get_alloc_size(c->buft, &w->t));
    if (!w->buf) return B200_STATUS_ALLOC_FAILED;
    w->buf->usage = GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
    w->t.buffer = w->buf;
    w->t.data = w->buf->iface.get_base(w->buf);
    w->buf->iface.init_tensor(w->buf, &w->t);
    w->buf->iface.set_tensor(w->buf, &w->t, data, 0, nbytes);
    auto old = c->weights.find(name);
    if (old != c->weights.end()) {
        c->backend->iface.synchronize(c->backend);
        old->second->buf->iface.free_buffer(old->second->buf);
    }
    c->weights[name] = std::move(w);
    c->graphs.clear();   // graphs hold pointers to the weight tensors
    c->last = nullptr;
    return B200_STATUS_SUCCESS;
}

int b200_llama_kv_clear(b200_llama *c) {
    B200_REQUIRE(c != nullptr, "llama_kv_clear: null context");
    c->backend->iface.synchronize(c->backend);
    c->kv_buf->iface.clear(c->kv_buf, 0);
    std::fill(c->cell_pos.begin(), c->cell_pos.end(), -1);
    std::fill(c->cell_seq.begin(), c->cell_seq.end(), -1);
    c->used = 0;
    return B200_STATUS_SUCCESS;
}

int32_t b200_llama_kv_used(const b200_llama *c) { return c ? c->used : 0; }

int b200_llama_get_hparams(const b200_llama *c, b200_llama_hparams *out) {
    B200_REQUIRE(c != nullptr && out != nullptr, "llama_get_hparams: null argument");
    *out = c->hp;
    return B200_STATUS_SUCCESS;
}

int b200_llama_decode(b200_llama *c, const int32_t *tokens, const int32_t *pos, int32_t n, float *logits, int32_t *argmax) {
    B200_REQUIRE(n > 0, "llama_decode: batch size %d out of (0, %d]", n, c ? c->n_batch : 0);
    const int32_t last = n - 1;
    return b200_llama_decode_seqs(c, tokens, pos, nullptr, n, &last, 1, logits, argmax);
}

int b200_llama_decode_seqs(b200_llama *c, const int32_t *tokens, const int32_t *pos, const int32_t *seq_ids, int32_t n,
                           const int32_t *out_rows, int32_t n_out, float *logits, int32_t *argmax) {
    B200_REQUIRE(c != nullptr && tokens != nullptr && pos != nullptr && out_rows != nullptr, "llama_decode: null argument");
    B200_REQUIRE(n > 0 && n <= c->n_batch, "llama_decode: batch size %d out of (0, %d]", n, c->n_batch);
    B200_REQUIRE(n_out > 0 && n_out <= n, "llama_decode: %d output rows for %d tokens", n_out, n);
    B200_REQUIRE(c->used + n <= c->n_ctx, "llama_decode: kv cache full (%d used + %d > %d)", c->used, n, c->n_ctx);
    for (int i = 0; i < n; i++)
        B200_REQUIRE(tokens[i] >= 0 && tokens[i] < c->hp.n_vocab, "llama_decode: token %d out of range", tokens[i]);
    for (int i = 0; i < n_out; i++) B200_REQUIRE(out_rows[i] >= 0 && out_rows[i] < n, "llama_decode: output row %d out of range", out_rows[i]);

    // find_slot + assign: the next free cells, in order; a cell remembers its sequence and position
    const int32_t head = c->used;
    const int64_t n_kv = n_kv_for(c, head + n);

    // the graph for this (n, n_kv, n_out), sized and built once
    auto key = std::make_pair((int64_t)n * 65536 + n_out, n_kv);
    auto it = c->graphs.find(key);
    if (it == c->graphs.end()) {
        if (!c->compute_buf) {
            Graph measure;
            int rc = build_graph(c, &measure, nullptr, c->n_batch, c->n_ctx, c->n_batch);
            if (rc != B200_STATUS_SUCCESS) return rc;
            c->compute_buf = c->buft->iface.alloc_buffer(c->buft, measure.bytes + ALIGN);
            if (!c->compute_buf) return B200_STATUS_ALLOC_FAILED;
            c->compute_buf->usage = GGML_BACKEND_BUFFER_USAGE_COMPUTE;
        }
        std::unique_ptr<Graph> g(new Graph());
        int rc = build_graph(c, g.get(), (uint8_t *)c->compute_buf->iface.get_base(c->compute_buf), n, n_kv, n_out);
        if (rc != B200_STATUS_SUCCESS) return rc;
        B200_REQUIRE(g->bytes <= c->compute_buf->size, "llama_decode: graph needs %zu bytes, compute buffer has %zu", g->bytes, c->compute_buf->size);
        it = c->graphs.emplace(key, std::move(g)).first;
    }
    Graph *g = it->second.get();

    for (int i = 0; i < n; i++) {
        c->cell_pos[head + i] = pos[i];
        c->cell_seq[head + i] = seq_ids ? seq_ids[i] : 0;
    }
    c->used = head + n;
    // crates/llama/src/graph.rs:704-724 fill_kq_mask_f16 with the sequence test of llama-kv-cache's set_input_kq_mask:
    // 0 where the cell belongs to the query's sequence and holds a position <= the query's, -inf elsewhere
    c->mask_host.assign((size_t)n * n_kv, 0xFC00);
    for (int i = 0; i < n; i++) {
        const int32_t s = seq_ids ? seq_ids[i] : 0;
        for (int64_t j = 0; j < c->used; j++)
            if (c->cell_seq[j] == s && c->cell_pos[j] >= 0 && c->cell_pos[j] <= pos[i]) c->mask_host[(size_t)i * n_kv + j] = 0;
    }
    c->idx_host.resize(n);
    for (int i = 0; i < n; i++) c->idx_host[i] = head + i;

    // inputs land with synchronous copies after the previous step has drained
    c->backend->iface.synchronize(c->backend);
    set_input_async(c->backend, g->tokens, tokens, (size_t)n * 4);
    set_input_async(c->backend, g->pos, pos, (size_t)n * 4);
    set_input_async(c->backend, g->mask, c->mask_host.data(), c->mask_host.size() * 2);
    set_input_async(c->backend, g->row_idx, c->idx_host.data(), (size_t)n * 8);
    set_input_async(c->backend, g->out_ids, out_rows, (size_t)n_out * 4);

    int rc = run_graph(c, g, (int)g->nodes.size() - (argmax ? 0 : 1));   // the ARGMAX node is last
    if (rc != B200_STATUS_SUCCESS) return rc;
    c->last = g;
    if (logits) c->backend->iface.get_tensor_async(c->backend, g->logits, logits, 0, (size_t)c->hp.n_vocab * n_out * 4);
    if (argmax) c->backend->iface.get_tensor_async(c->backend, g->argmax, argmax, 0, (size_t)n_out * 4);
    c->backend->iface.synchronize(c->backend);
    int code = 0;
    rc = b200_kernel_error(&code);
    if (rc != B200_STATUS_SUCCESS) return rc;
    B200_REQUIRE(code == 0, "llama_decode: a kernel reported error code %d", code);
    return B200_STATUS_SUCCESS;
}

int b200_llama_read_node(b200_llama *c, const char *name, void *out, size_t nbytes) {
    B200_REQUIRE(c != nullptr && name != nullptr && out != nullptr, "llama_read_node: null argument");
    B200_REQUIRE(c->last != nullptr, "llama_read_node: no decode call yet");
    const ggml_tensor *found = nullptr;
    for (const ggml_tensor &t : c->last->tensors)
        if (strcmp(t.name, name) == 0) found = &t;
    B200_REQUIRE(found != nullptr, "llama_read_node: no tensor named %s", name);
    B200_REQUIRE(nbytes <= found->nb[3], "llama_read_node: %s holds %zu bytes, %zu asked", name, found->nb[3], nbytes);
    c->backend->iface.get_tensor_async(c->backend, found, out, 0, nbytes);
    c->backend->iface.synchronize(c->backend);
    return B200_STATUS_SUCCESS;
}

int b200_llama_replay(b200_llama *c, int32_t reps, float *ms) {
    B200_REQUIRE(c != nullptr && ms != nullptr && reps > 0, "llama_replay: bad argument");
    B200_REQUIRE(c->last != nullptr, "llama_replay: no decode call to replay");
    Graph *g = c->last;
    void *e0 = nullptr, *e1 = nullptr;
    int rc = b200_event_create(&e0);
    if (rc == B200_STATUS_SUCCESS) rc = b200_event_create(&e1);
    if (rc == B200_STATUS_SUCCESS) rc = b200_event_record(e0, c->stream);
    for (int i = 0; i < reps && rc == B200_STATUS_SUCCESS; i++) rc = run_graph(c, g, (int)g->nodes.size() - 1);
    if (rc == B200_STATUS_SUCCESS) rc = b200_event_record(e1, c->stream);
    if (rc == B200_STATUS_SUCCESS) rc = b200_event_synchronize(e1);
    if (rc == B200_STATUS_SUCCESS) rc = b200_event_elapsed_ms(e0, e1, ms);
    if (e0) b200_event_destroy(e0);
    if (e1) b200_event_destroy(e1);
    return rc;
}

}  // extern "C"
