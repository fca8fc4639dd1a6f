// The ggml backend plug-in face: registry, device, buffer type, buffer and backend vtables
// (include/ggml_b200_backend.h), on top of the op-level entry points.
//
// What the reference's scheduler expects of a backend (crates/ggml/src/backend_sched.rs:884-989,
// 1746-1752): supports_op / supports_buft answer per node, buffers hold the tensors the nodes read and
// write, graph_compute gets one split's nodes and returns a ggml status.  Quantized tensors that live
// in a buffer of this backend are kept in the 32-row tile layout: set_tensor re-orders the ggml blocks
// on the way in, get_tensor on the way out, get_alloc_size reports the padded size.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "ggml_b200_backend.h"

namespace b200 {
namespace {

// ---- type table (crates/ggml/src/types.rs:15-53,172) -----------------------------------------
struct TypeTraits { int blck; int size; };
static TypeTraits traits(int type) {
    switch (type) {
        case B200_TYPE_F32: return {1, 4};
        case B200_TYPE_F16: return {1, 2};
        case B200_TYPE_Q4_0: return {32, 18};
        case B200_TYPE_Q8_0: return {32, 34};
        case B200_TYPE_Q4_K: return {256, 144};
        case B200_TYPE_Q6_K: return {256, 210};
        case B200_TYPE_Q8_K: return {256, 292};
        case B200_TYPE_I32: return {1, 4};
        case B200_TYPE_I64: return {1, 8};
        case B200_TYPE_MXFP4: return {32, 17};
        default: return {0, 0};
    }
}
static size_t row_size(int type, int64_t ne0) {
    TypeTraits t = traits(type);
    return t.blck ? (size_t)(ne0 / t.blck) * t.size : 0;
}
static size_t ggml_nbytes(const ggml_tensor *t) {
    TypeTraits tr = traits(t->type);
    if (!tr.blck) return 0;
    for (int i = 0; i < 4; i++)
        if (t->ne[i] <= 0) return 0;
    size_t n = (size_t)t->ne[0] * t->nb[0] / tr.blck;
    for (int i = 1; i < 4; i++) n += (size_t)(t->ne[i] - 1) * t->nb[i];
    return n;
}
static bool is_contiguous(const ggml_tensor *t) {
    TypeTraits tr = traits(t->type);
    if (!tr.blck) return false;
    if (t->nb[0] != (size_t)tr.size) return false;
    if (t->nb[1] != row_size(t->type, t->ne[0])) return false;
    return t->nb[2] == t->nb[1] * t->ne[1] && t->nb[3] == t->nb[2] * t->ne[2];
}
// a quantized tensor this backend keeps in tile layout: [k, n rows, n_expert, 1]
static bool is_tiled_tensor(const ggml_tensor *t) {
    return is_quant_type(t->type) && t->ne[0] % GROUP_K == 0 && t->ne[3] == 1 && t->view_src == nullptr;
}
static size_t tiled_expert_bytes(const ggml_tensor *t) { return b200_weight_nbytes(t->type, t->ne[1], t->ne[0]); }

// ---- contexts -----------------------------------------------------------------------------------
struct DeviceCtx {
    int index;
    std::string name, description;
};
struct BufferCtx {
    int device;
    void *base;
    std::string error;   // set by the void-returning vtable entries, reported by graph_compute
};
struct BackendCtx {
    int device;
    cudaStream_t stream;
    int cpu_threads;
    std::string name;
};

static std::mutex g_mu;
static std::vector<ggml_backend_device *> g_devices;
static std::vector<ggml_backend_buffer_type *> g_bufts;
static ggml_backend_reg g_reg;
static bool g_reg_ready = false;

static int dev_of(ggml_backend_dev_t d) { return ((DeviceCtx *)d->context)->index; }
static BufferCtx *bctx(ggml_backend_buffer_t b) { return (BufferCtx *)b->context; }
static void note(BufferCtx *c, const char *what) {
    if (c->error.empty()) c->error = std::string(what) + ": " + b200_last_error();
}

// ---- buffer -------------------------------------------------------------------------------------
static void buf_free(ggml_backend_buffer_t b) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (c->base) cudaFree(c->base);
    delete c;
    delete b;
}
static void *buf_get_base(ggml_backend_buffer_t b) { return bctx(b)->base; }
static int buf_init_tensor(ggml_backend_buffer_t, ggml_tensor *) { return B200_STATUS_SUCCESS; }

static void buf_memset_tensor(ggml_backend_buffer_t b, ggml_tensor *t, uint8_t value, size_t offset, size_t size) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (b200_memset((uint8_t *)t->data + offset, value, size, nullptr) != B200_STATUS_SUCCESS) note(c, "memset_tensor");
    cudaStreamSynchronize(nullptr);
}

// rows [r0, r0 + nr) of expert e of a tiled tensor, whole rows only, r0 on a tile boundary
static int tiled_rows_io(const ggml_tensor *t, size_t offset, size_t size, int64_t *e, int64_t *r0, int64_t *nr) {
    const size_t rs = row_size(t->type, t->ne[0]);
    const size_t per_expert = rs * t->ne[1];
    B200_REQUIRE(rs > 0 && offset % rs == 0 && size % rs == 0, "tiled tensor i/o must cover whole rows (offset %zu size %zu row %zu)",
                 offset, size, rs);
    *e = (int64_t)(offset / per_expert);
    const size_t in_e = offset % per_expert;
    *r0 = (int64_t)(in_e / rs);
    *nr = (int64_t)(size / rs);
    B200_REQUIRE(*r0 % TILE_ROWS == 0, "tiled tensor i/o must start on a 32-row boundary (row %lld)", (long long)*r0);
    B200_REQUIRE(*r0 + *nr <= t->ne[1] || *r0 == 0, "tiled tensor i/o crosses an expert boundary mid-way");
    return B200_STATUS_SUCCESS;
}

static int tiled_io(const ggml_tensor *t, void *host, size_t offset, size_t size, bool upload) {
    int64_t e, r0, nr;
    int rc = tiled_rows_io(t, offset, size, &e, &r0, &nr);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const size_t rs = row_size(t->type, t->ne[0]);
    const size_t eb = tiled_expert_bytes(t);
    const int64_t groups = t->ne[0] / GROUP_K;
    uint8_t *h = (uint8_t *)host;
    // a piece may span several experts when it starts at an expert's first row
    while (nr > 0) {
        const int64_t take = std::min<int64_t>(nr, t->ne[1] - r0);
        uint8_t *dev = (uint8_t *)t->data + (size_t)e * eb + (size_t)(r0 / TILE_ROWS) * groups * chunk_bytes(t->type);
        rc = upload ? b200_weight_upload(t->type, take, t->ne[0], h, dev, nullptr)
                    : b200_weight_download(t->type, take, t->ne[0], dev, h, nullptr);
        if (rc != B200_STATUS_SUCCESS) return rc;
        h += (size_t)take * rs;
        nr -= take;
        r0 = 0;
        e++;
    }
    return B200_STATUS_SUCCESS;
}

static void buf_set_tensor(ggml_backend_buffer_t b, ggml_tensor *t, const void *data, size_t offset, size_t size) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (size == 0) return;
    if (is_tiled_tensor(t)) {
        if (tiled_io(t, const_cast<void *>(data), offset, size, true) != B200_STATUS_SUCCESS) note(c, "set_tensor");
        return;
    }
    if (b200_memcpy_h2d((uint8_t *)t->data + offset, data, size, nullptr) != B200_STATUS_SUCCESS) note(c, "set_tensor");
    cudaStreamSynchronize(nullptr);
}
static void buf_get_tensor(ggml_backend_buffer_t b, const ggml_tensor *t, void *data, size_t offset, size_t size) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (size == 0) return;
    if (is_tiled_tensor(t)) {
        if (tiled_io(t, data, offset, size, false) != B200_STATUS_SUCCESS) note(c, "get_tensor");
        return;
    }
    if (b200_memcpy_d2h(data, (const uint8_t *)t->data + offset, size, nullptr) != B200_STATUS_SUCCESS) note(c, "get_tensor");
}
static bool buf_cpy_tensor(ggml_backend_buffer_t b, const ggml_tensor *src, ggml_tensor *dst) {
    // same-layout device-to-device copy between two buffers of this backend
    if (!src->buffer || src->buffer->iface.get_base != buf_get_base) return false;
    if (src->type != dst->type || !is_contiguous(src) || !is_contiguous(dst)) return false;
    for (int i = 0; i < 4; i++)
        if (src->ne[i] != dst->ne[i]) return false;
    BufferCtx *c = bctx(b);
    if (bctx(src->buffer)->device != c->device) return false;
    cudaSetDevice(c->device);
    const size_t n = is_tiled_tensor(src) ? tiled_expert_bytes(src) * src->ne[2] : ggml_nbytes(src);
    return cudaMemcpy(dst->data, src->data, n, cudaMemcpyDeviceToDevice) == cudaSuccess;
}
static void buf_clear(ggml_backend_buffer_t b, uint8_t value) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (c->base) cudaMemset(c->base, value, b->size);
}

// ---- buffer type ----------------------------------------------------------------------------------
static const char *buft_get_name(ggml_backend_buffer_type_t t) { return ((DeviceCtx *)t->device->context)->name.c_str(); }
static ggml_backend_buffer_t buft_alloc(ggml_backend_buffer_type_t t, size_t size) {
    const int dev = dev_of(t->device);
    if (cudaSetDevice(dev) != cudaSuccess) return nullptr;
    void *p = nullptr;
    if (size > 0 && cudaMalloc(&p, size) != cudaSuccess) {
        cudaGetLastError();
        set_error("alloc_buffer: cudaMalloc of %zu bytes failed on device %d", size, dev);
        return nullptr;
    }
    ggml_backend_buffer *b = new ggml_backend_buffer();
    memset(&b->iface, 0, sizeof(b->iface));
    b->iface.free_buffer = buf_free;
    b->iface.get_base = buf_get_base;
    b->iface.init_tensor = buf_init_tensor;
    b->iface.memset_tensor = buf_memset_tensor;
    b->iface.set_tensor = buf_set_tensor;
    b->iface.get_tensor = buf_get_tensor;
    b->iface.cpy_tensor = buf_cpy_tensor;
    b->iface.clear = buf_clear;
    b->buft = t;
    b->context = new BufferCtx{dev, p, std::string()};
    b->size = size;
    b->usage = GGML_BACKEND_BUFFER_USAGE_ANY;
    return b;
}
static size_t buft_alignment(ggml_backend_buffer_type_t) { return 256; }
static size_t buft_max_size(ggml_backend_buffer_type_t) { return SIZE_MAX; }
static size_t buft_alloc_size(ggml_backend_buffer_type_t, const ggml_tensor *t) {
    if (is_tiled_tensor(t)) return tiled_expert_bytes(t) * (size_t)t->ne[2];
    return ggml_nbytes(t);
}
static bool buft_is_host(ggml_backend_buffer_type_t) { return false; }

// ---- supports_op ----------------------------------------------------------------------------------
static bool in_our_buffer(const ggml_tensor *t) { return t && t->buffer && t->buffer->iface.get_base == buf_get_base; }

static bool supports_mul_mat(const ggml_tensor *op, std::string *why) {
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    auto no = [&](const char *m) { if (why) *why = m; return false; };
    if (!w || !x) return no("missing source");
    if (!is_quant_type(w->type)) return no("weight type is not one of Q4_0, Q8_0, Q4_K, Q6_K, MXFP4");
    if (w->ne[0] % GROUP_K) return no("k is not a multiple of 256");
    if (w->view_src || !is_contiguous(w) || w->ne[3] != 1) return no("weights must be plain contiguous rows");
    if (x->type != B200_TYPE_F32 || op->type != B200_TYPE_F32) return no("activations and result must be F32");
    if (x->nb[0] != 4 || op->nb[0] != 4 || x->nb[1] % 4 || op->nb[1] % 4) return no("activation rows must be dense f32");
    if (x->ne[0] != w->ne[0] || op->ne[0] != w->ne[1]) return no("shape mismatch");
    if (op->op == GGML_OP_MUL_MAT) {
        if (w->ne[2] != 1) return no("batched weights are not supported");
        if (op->ne[1] != x->ne[1] || op->ne[2] != x->ne[2] || op->ne[3] != x->ne[3]) return no("shape mismatch");
    } else {
        const ggml_tensor *ids = op->src[2];
        if (!ids || ids->type != B200_TYPE_I32) return no("ids must be I32");
        if (!is_contiguous(ids) || !is_contiguous(x) || !is_contiguous(op)) return no("mul_mat_id operands must be contiguous");
        if (op->ne[1] != ids->ne[0] || op->ne[2] != ids->ne[1] || x->ne[2] != ids->ne[1]) return no("shape mismatch");
    }
    return true;
}

static bool supports_flash(const ggml_tensor *op, std::string *why) {
    const ggml_tensor *q = op->src[0], *k = op->src[1], *v = op->src[2], *m = op->src[3];
    auto no = [&](const char *msg) { if (why) *why = msg; return false; };
    if (!q || !k || !v) return no("missing source");
    if (q->type != B200_TYPE_F32 || k->type != B200_TYPE_F16 || v->type != B200_TYPE_F16) return no("q must be F32, k and v F16");
    if (q->ne[3] != 1 || k->ne[3] != 1 || v->ne[3] != 1) return no("batch dimension must be 1");
    if ((q->ne[0] != 64 && q->ne[0] != 128) || (v->ne[0] != 64 && v->ne[0] != 128) || k->ne[0] != q->ne[0])
        return no("head sizes must be 64 or 128");
    if (q->nb[0] != 4 || k->nb[0] != 2 || v->nb[0] != 2) return no("rows must be dense");
    if (k->nb[1] % 16 || k->nb[2] % 16 || v->nb[1] % 16 || v->nb[2] % 16) return no("k/v rows must be 16-byte aligned");
    if (k->ne[1] != v->ne[1] || k->ne[2] != v->ne[2] || q->ne[2] % k->ne[2]) return no("head / length mismatch");
    if (m && (m->type != B200_TYPE_F16 || m->nb[0] != 2 || m->ne[0] < k->ne[1] || m->ne[1] < q->ne[1] || m->ne[2] != 1))
        return no("mask must be dense F16 [n_kv, n_tok]");
    return true;
}

static bool op_supported(const ggml_tensor *op, std::string *why) {
    switch (op->op) {
        case GGML_OP_NONE: case GGML_OP_RESHAPE: case GGML_OP_VIEW: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE:
            return true;
        case GGML_OP_MUL_MAT: case GGML_OP_MUL_MAT_ID: return supports_mul_mat(op, why);
        case GGML_OP_FLASH_ATTN_EXT: return supports_flash(op, why);
        default:
            if (why) *why = "op is outside the quantized mat-mul / flash-attention path";
            return false;
    }
}

// ---- graph_compute ----------------------------------------------------------------------------------
static int compute_mul_mat(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    const int64_t k = w->ne[0], n = w->ne[1], m = x->ne[1];
    for (int64_t i3 = 0; i3 < x->ne[3]; i3++)
        for (int64_t i2 = 0; i2 < x->ne[2]; i2++) {
            const float *xp = (const float *)((const uint8_t *)x->data + i2 * x->nb[2] + i3 * x->nb[3]);
            float *dp = (float *)((uint8_t *)op->data + i2 * op->nb[2] + i3 * op->nb[3]);
            int rc = b200_mul_mat(w->type, n, k, m, w->data, xp, (int64_t)(x->nb[1] / 4), dp, (int64_t)(op->nb[1] / 4),
                                  B200_ROUTE_AUTO, bc->stream);
            if (rc != B200_STATUS_SUCCESS) return rc;
        }
    return B200_STATUS_SUCCESS;
}
static int compute_mul_mat_id(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *w = op->src[0], *x = op->src[1], *ids = op->src[2];
    return b200_mul_mat_id(w->type, w->ne[1], w->ne[0], w->ne[2], x->ne[1], x->ne[2], ids->ne[0], w->data,
                           (const float *)x->data, (const int32_t *)ids->data, (float *)op->data, B200_ROUTE_AUTO, bc->stream);
}
static int compute_flash(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *q = op->src[0], *k = op->src[1], *v = op->src[2], *m = op->src[3], *s = op->src[4];
    B200_REQUIRE(is_contiguous(op), "flash_attn_ext: dst must be contiguous");
    b200_flash_attn_args a;
    memset(&a, 0, sizeof(a));
    a.dk = q->ne[0]; a.dv = v->ne[0]; a.n_tok = q->ne[1]; a.n_head = q->ne[2]; a.n_head_kv = k->ne[2]; a.n_kv = k->ne[1];
    a.q = (const float *)q->data; a.q_nb1 = (int64_t)q->nb[1]; a.q_nb2 = (int64_t)q->nb[2];
    a.k = k->data; a.k_nb1 = (int64_t)k->nb[1]; a.k_nb2 = (int64_t)k->nb[2];
    a.v = v->data; a.v_nb1 = (int64_t)v->nb[1]; a.v_nb2 = (int64_t)v->nb[2];
    a.mask = m ? m->data : nullptr; a.mask_nb1 = m ? (int64_t)m->nb[1] : 0;
    a.sinks = s ? (const float *)s->data : nullptr;
    memcpy(&a.scale, &op->op_params[0], 4);
    memcpy(&a.max_bias, &op->op_params[1], 4);
    memcpy(&a.logit_softcap, &op->op_params[2], 4);
    a.dst = (float *)op->data;
    a.n_chunks = bc->cpu_threads;
    a.mode = 0;
    return b200_flash_attn_ext(&a, bc->stream);
}

static int backend_graph_compute(ggml_backend_t be, ggml_cgraph *g) {
    BackendCtx *bc = (BackendCtx *)be->context;
    B200_REQUIRE(g != nullptr && (g->n_nodes == 0 || g->nodes != nullptr), "graph_compute: null graph");
    B200_CUDA(cudaSetDevice(bc->device));
    for (int i = 0; i < g->n_nodes; i++) {
        const ggml_tensor *op = g->nodes[i];
        B200_REQUIRE(op != nullptr, "graph_compute: node %d is null", i);
        std::string why;
        if (!op_supported(op, &why)) {
            set_error("graph_compute: node %d '%s' (op %d) is not supported: %s", i, op->name, op->op, why.c_str());
            return B200_STATUS_BACKEND_ERROR;
        }
        for (int s = 0; s < GGML_MAX_SRC; s++) {
            const ggml_tensor *src = op->src[s];
            if (src && src->buffer && in_our_buffer(src) && !bctx(src->buffer)->error.empty()) {
                set_error("graph_compute: source '%s' of node %d failed earlier: %s", src->name, i, bctx(src->buffer)->error.c_str());
                return B200_STATUS_BACKEND_ERROR;
            }
        }
        int rc = B200_STATUS_SUCCESS;
        switch (op->op) {
            case GGML_OP_MUL_MAT: rc = compute_mul_mat(bc, op); break;
            case GGML_OP_MUL_MAT_ID: rc = compute_mul_mat_id(bc, op); break;
            case GGML_OP_FLASH_ATTN_EXT: rc = compute_flash(bc, op); break;
            default: break;   // views and leaves: nothing to run
        }
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    return B200_STATUS_SUCCESS;
}

// ---- backend -------------------------------------------------------------------------------------
static const char *backend_get_name(ggml_backend_t be) { return ((BackendCtx *)be->context)->name.c_str(); }
static void backend_free(ggml_backend_t be) {
    BackendCtx *bc = (BackendCtx *)be->context;
    cudaSetDevice(bc->device);
    cudaStreamSynchronize(bc->stream);
    delete bc;
    delete be;
}
static void backend_set_tensor_async(ggml_backend_t, ggml_tensor *t, const void *data, size_t offset, size_t size) {
    if (t->buffer) t->buffer->iface.set_tensor(t->buffer, t, data, offset, size);
}
static void backend_get_tensor_async(ggml_backend_t be, const ggml_tensor *t, void *data, size_t offset, size_t size) {
    BackendCtx *bc = (BackendCtx *)be->context;
    cudaSetDevice(bc->device);
    cudaStreamSynchronize(bc->stream);
    if (t->buffer) t->buffer->iface.get_tensor(t->buffer, t, data, offset, size);
}
static void backend_synchronize(ggml_backend_t be) {
    BackendCtx *bc = (BackendCtx *)be->context;
    cudaSetDevice(bc->device);
    cudaStreamSynchronize(bc->stream);
}
static void backend_set_cpu_threads(ggml_backend_t be, int n) {
    if (be && n > 0) ((BackendCtx *)be->context)->cpu_threads = n;
}

// ---- device ---------------------------------------------------------------------------------------
static const char *dev_get_name(ggml_backend_dev_t d) { return ((DeviceCtx *)d->context)->name.c_str(); }
static const char *dev_get_description(ggml_backend_dev_t d) { return ((DeviceCtx *)d->context)->description.c_str(); }
static void dev_get_memory(ggml_backend_dev_t d, size_t *free_b, size_t *total_b) {
    size_t f = 0, t = 0;
    b200_device_info(dev_of(d), nullptr, 0, &f, &t, nullptr, nullptr, nullptr);
    if (free_b) *free_b = f;
    if (total_b) *total_b = t;
}
static int dev_get_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_GPU; }
static void dev_get_props(ggml_backend_dev_t d, ggml_backend_dev_props *p) {
    p->name = dev_get_name(d);
    p->description = dev_get_description(d);
    dev_get_memory(d, &p->memory_free, &p->memory_total);
    p->type = GGML_BACKEND_DEVICE_TYPE_GPU;
    p->device_id = nullptr;
    p->caps = {false, false, false, false, false};
}
static ggml_backend_t dev_init_backend(ggml_backend_dev_t d, const char *params) {
    const int dev = dev_of(d);
    if (cudaSetDevice(dev) != cudaSuccess) {
        set_error("init_backend: cannot select CUDA device %d", dev);
        return nullptr;
    }
    BackendCtx *bc = new BackendCtx{dev, nullptr, 8, std::string("B200") + std::to_string(dev)};
    if (params) {   // "cpu_threads=<n>"
        const char *p = strstr(params, "cpu_threads=");
        if (p) {
            int n = atoi(p + 12);
            if (n > 0) bc->cpu_threads = n;
        }
    }
    ggml_backend *be = new ggml_backend();
    memset(&be->iface, 0, sizeof(be->iface));
    be->guid = (void *)"b200-ggml-backend";
    be->iface.get_name = backend_get_name;
    be->iface.free = backend_free;
    be->iface.set_tensor_async = backend_set_tensor_async;
    be->iface.get_tensor_async = backend_get_tensor_async;
    be->iface.synchronize = backend_synchronize;
    be->iface.graph_compute = backend_graph_compute;
    be->device = d;
    be->context = bc;
    return be;
}
static ggml_backend_buffer_type_t dev_get_buffer_type(ggml_backend_dev_t d) { return g_bufts[dev_of(d)]; }
static bool dev_supports_op(ggml_backend_dev_t, const ggml_tensor *op) { return op && op_supported(op, nullptr); }
static bool dev_supports_buft(ggml_backend_dev_t d, ggml_backend_buffer_type_t t) { return t == g_bufts[dev_of(d)]; }
static bool dev_offload_op(ggml_backend_dev_t, const ggml_tensor *op) {
    // weights in host memory: worth taking only for batches (the CUDA backend's own rule of thumb)
    return op && (op->op == GGML_OP_MUL_MAT || op->op == GGML_OP_MUL_MAT_ID) && op->ne[1] >= 32;
}

// ---- registry -------------------------------------------------------------------------------------
static int usable_device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int ok = 0;
    for (int i = 0; i < n; i++) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess && major == 10) ok = i + 1;
    }
    return ok;   // devices [0, ok) are exposed; the kernels are sm_100a only
}
static const char *reg_get_name(ggml_backend_reg_t) { return "B200"; }
static size_t reg_get_device_count(ggml_backend_reg_t) { return g_devices.size(); }
static ggml_backend_dev_t reg_get_device(ggml_backend_reg_t, size_t i) { return i < g_devices.size() ? g_devices[i] : nullptr; }
static void *reg_get_proc_address(ggml_backend_reg_t, const char *name) {
    if (name && strcmp(name, "b200_backend_set_cpu_threads") == 0) return (void *)backend_set_cpu_threads;
    return nullptr;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int ggml_backend_score(void) { return usable_device_count() > 0 ? 100 : 0; }

extern "C" ggml_backend_reg_t ggml_backend_init(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_reg_ready) return &g_reg;
    g_reg.api_version = GGML_BACKEND_API_VERSION;
    memset(&g_reg.iface, 0, sizeof(g_reg.iface));
    g_reg.iface.get_name = reg_get_name;
    g_reg.iface.get_device_count = reg_get_device_count;
    g_reg.iface.get_device = reg_get_device;
    g_reg.iface.get_proc_address = reg_get_proc_address;
    g_reg.context = nullptr;
    const int n = usable_device_count();
    for (int i = 0; i < n; i++) {
        char nm[256] = "";
        b200_device_info(i, nm, sizeof(nm), nullptr, nullptr, nullptr, nullptr, nullptr);
        ggml_backend_device *d = new ggml_backend_device();
        memset(&d->iface, 0, sizeof(d->iface));
        d->iface.get_name = dev_get_name;
        d->iface.get_description = dev_get_description;
        d->iface.get_memory = dev_get_memory;
        d->iface.get_type = dev_get_type;
        d->iface.get_props = dev_get_props;
        d->iface.init_backend = dev_init_backend;
        d->iface.get_buffer_type = dev_get_buffer_type;
        d->iface.supports_op = dev_supports_op;
        d->iface.supports_buft = dev_supports_buft;
        d->iface.offload_op = dev_offload_op;
        d->reg = &g_reg;
        d->context = new DeviceCtx{i, std::string("B200") + std::to_string(i), std::string(nm)};
        g_devices.push_back(d);
        ggml_backend_buffer_type *t = new ggml_backend_buffer_type();
        t->iface.get_name = buft_get_name;
        t->iface.alloc_buffer = buft_alloc;
        t->iface.get_alignment = buft_alignment;
        t->iface.get_max_size = buft_max_size;
        t->iface.get_alloc_size = buft_alloc_size;
        t->iface.is_host = buft_is_host;
        t->device = d;
        t->context = nullptr;
        g_bufts.push_back(t);
    }
    g_reg_ready = true;
    return &g_reg;
}
