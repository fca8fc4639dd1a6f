// The ggml backend plug-in face: registry, device, buffer type, buffer and backend vtables
// (include/ggml_b200_backend.h), on top of the op-level entry points.
//
// What the reference's scheduler expects of a backend (crates/ggml/src/backend_sched.rs:884-989,
// 1746-1752): supports_op / supports_buft answer per node, buffers hold the tensors the nodes read and
// write, graph_compute gets one split's nodes and returns a ggml status.  Quantized tensors that live
// in a buffer of this backend are kept in the 32-row tile layout: set_tensor re-orders the ggml blocks
// on the way in, get_tensor on the way out, get_alloc_size reports the padded size.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "ggml_b200_backend.h"
#include "tp.h"
#include "decode_persistent.h"

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
    // Host copies of the small I32 tensors written through set_tensor (token positions), keyed by the
    // tensor's data pointer: ROPE builds its cos/sin table on the host from them without a read-back.
    std::mutex mu;
    std::unordered_map<const void *, std::vector<int32_t>> i32_shadow;
};
struct BackendCtx {
    int device;
    cudaStream_t stream;
    int cpu_threads;
    std::string name;
    int silu_wide;                  // 1: reproduce an AVX512 host's SILU (crates/ggml/src/simd_x86.rs:1028-1038)
    // the quantized activations of the last MUL_MAT, reused while the next ones read the same rows
    void *act = nullptr;
    size_t act_bytes = 0;
    const void *act_src = nullptr;
    int64_t act_m = 0, act_k = 0, act_ld = 0;
    int act_kind = 0;
    // ROPE tables.  by_pos: one row per position 0 .. rows-1 for a parameter set, indexed on the device
    // by the position tensor, so that a step's launches do not depend on the positions' values (a few
    // parameter sets are kept).  per_tok: the fallback for positions such a table cannot hold, one row
    // per token of the current node.
    struct RopeTable {
        std::vector<int32_t> key;   // op_params, head size, frequency-factor bits
        float *dev = nullptr;
        int64_t rows = 0;
        uint64_t used = 0;
    };
    std::vector<RopeTable> rope_by_pos;
    uint64_t rope_clock = 0;
    float *rope_dev = nullptr;
    size_t rope_dev_floats = 0;
    std::vector<float> rope_host;
    std::vector<int32_t> rope_key;
    // CUDA graphs of node lists seen before: the second time a list comes by unchanged it is captured,
    // afterwards replayed.  generation counts the re-allocations that make captured addresses stale.
    struct CapturedGraph {
        uint64_t key = 0;
        cudaGraphExec_t exec = nullptr;
        uint64_t generation = 0;
        unsigned long long scratch_generation = 0;
        bool refused = false;     // a capture attempt failed: run this list eagerly from now on
        uint64_t used = 0;
    };
    std::vector<CapturedGraph> captured;
    uint64_t generation = 0;
    bool graphs_enabled = true;
    bool fuse_glue = true;          // one launch for neighbouring ROPE / SET_ROWS nodes (B200_FUSE_GLUE=0 / fuse_glue=0: off)
    bool fuse_siblings = true;      // one launch for one-row Q4_K mat-muls over the same activations (B200_FUSE_SIBLINGS=0 / fuse_siblings=0: off)
    bool fuse_prologue = true;      // the norm / silu / quantization in front of a one-row Q4_K mat-mul inside its kernel (B200_FUSE_PROLOGUE=0 / fuse_prologue=0: off)
    bool capturable = true;       // cleared by a node that had to talk to the device while being issued
    // One-token steps recognized as a whole (see match_decode_step): the phase list of the persistent kernel, on the device
    struct StepPlan {
        uint64_t key = 0;
        bool usable = false;        // false: the list was looked at and is not a step the kernel takes
        int first = 0, last = 0;    // nodes [first, last) are the kernel's
        int n_phases = 0;
        DpPhase *dev_phases = nullptr;
        DpSync *dev_sync = nullptr;
        float *dev_partial = nullptr;
        uint64_t generation = 0;
        uint64_t used = 0;
    };
    std::vector<StepPlan> plans;
    bool persistent_decode = false; // B200_DECODE_PERSISTENT=1 / decode_persistent=1: on
    uint64_t current_key = 0;       // node_list_key of the list being computed (0: not known)
    TpGroup *tp = nullptr;        // the tensor-parallel group whose collectives the TP_* nodes run (owned by the driver)
};
constexpr size_t SHADOW_MAX_BYTES = 1 << 20;
constexpr int64_t ROPE_TABLE_MIN_ROWS = 4096, ROPE_TABLE_MAX_ROWS = 1 << 20;
constexpr size_t ROPE_TABLES_KEPT = 4, GRAPHS_KEPT = 512;   // a tensor-parallel step is ~2 node lists per layer

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

static void shadow_drop(BufferCtx *c, const void *data) {
    std::lock_guard<std::mutex> lk(c->mu);
    c->i32_shadow.erase(data);
}
static void buf_memset_tensor(ggml_backend_buffer_t b, ggml_tensor *t, uint8_t value, size_t offset, size_t size) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (t->type == B200_TYPE_I32) shadow_drop(c, t->data);
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

// small I32 tensors (positions) keep a host copy of what was last written to them
static void shadow_note_write(BufferCtx *c, const ggml_tensor *t, const void *data, size_t offset, size_t size) {
    if (t->type == B200_TYPE_I32 && ggml_nbytes(t) <= SHADOW_MAX_BYTES && offset % 4 == 0 && size % 4 == 0 &&
        offset + size <= ggml_nbytes(t) && is_contiguous(t)) {
        std::lock_guard<std::mutex> lk(c->mu);
        std::vector<int32_t> &sh = c->i32_shadow[t->data];
        const bool fresh = sh.size() != ggml_nbytes(t) / 4;
        if (fresh && (offset != 0 || size != ggml_nbytes(t))) {
            c->i32_shadow.erase(t->data);   // a partial write into a tensor whose other values are unknown here
        } else {
            sh.resize(ggml_nbytes(t) / 4);
            memcpy((uint8_t *)sh.data() + offset, data, size);
        }
    }
}
static void buf_set_tensor(ggml_backend_buffer_t b, ggml_tensor *t, const void *data, size_t offset, size_t size) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    if (size == 0) return;
    if (is_tiled_tensor(t)) {
        if (tiled_io(t, const_cast<void *>(data), offset, size, true) != B200_STATUS_SUCCESS) note(c, "set_tensor");
        cudaStreamSynchronize(nullptr);   // set_tensor is synchronous: the re-ordering kernel has finished on return
        return;
    }
    shadow_note_write(c, t, data, offset, size);
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
    if (dst->type == B200_TYPE_I32) shadow_drop(c, dst->data);
    const size_t n = is_tiled_tensor(src) ? tiled_expert_bytes(src) * src->ne[2] : ggml_nbytes(src);
    return cudaMemcpy(dst->data, src->data, n, cudaMemcpyDeviceToDevice) == cudaSuccess;
}
static void buf_clear(ggml_backend_buffer_t b, uint8_t value) {
    BufferCtx *c = bctx(b);
    cudaSetDevice(c->device);
    {
        std::lock_guard<std::mutex> lk(c->mu);
        c->i32_shadow.clear();
    }
    if (c->base) cudaMemset(c->base, value, b->size);
    cudaStreamSynchronize(nullptr);   // backends run on their own streams: the fill must have landed before they start
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
    BufferCtx *bc = new BufferCtx();
    bc->device = dev;
    bc->base = p;
    b->context = bc;
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

// rows of an F32 tensor addressed as base + r * nb[1]: dims above 1 must stack contiguously on dim 1
static bool f32_rows(const ggml_tensor *t) {
    return t && t->type == B200_TYPE_F32 && t->nb[0] == 4 && t->nb[1] % 4 == 0 && t->nb[2] == t->nb[1] * (size_t)t->ne[1] &&
           t->nb[3] == t->nb[2] * (size_t)t->ne[2];
}
static int64_t nrows_of(const ggml_tensor *t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
static bool same_shape(const ggml_tensor *a, const ggml_tensor *b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}

static bool supports_glue(const ggml_tensor *op, std::string *why) {
    auto no = [&](const char *m) { if (why) *why = m; return false; };
    const ggml_tensor *a = op->src[0], *b = op->src[1];
    switch (op->op) {
        case GGML_OP_RMS_NORM:
            if (!f32_rows(a) || !f32_rows(op) || !same_shape(a, op)) return no("rms_norm wants dense F32 rows");
            return true;
        case GGML_OP_ADD: case GGML_OP_MUL:
            if (!f32_rows(a) || !f32_rows(b) || !f32_rows(op) || !same_shape(a, op)) return no("add/mul want dense F32 rows");
            if (same_shape(a, b)) return true;
            // one row (or one element per row position) broadcast over every row of a
            if (b->ne[1] * b->ne[2] * b->ne[3] == 1 && a->ne[0] % b->ne[0] == 0) return true;
            return no("add/mul: src1 must match src0 or be a single row");
        case GGML_OP_UNARY:
            if (op->op_params[0] != GGML_UNARY_OP_SILU) return no("only SILU of the unary ops");
            if (!f32_rows(a) || !f32_rows(op) || !same_shape(a, op)) return no("silu wants dense F32 rows");
            return true;
        case GGML_OP_ROPE: {
            if (!a || !b || a->type != B200_TYPE_F32 || op->type != B200_TYPE_F32 || a->nb[0] != 4 || op->nb[0] != 4) return no("rope wants F32");
            if (!same_shape(a, op) || a->ne[3] != 1) return no("rope: shape");
            if (b->type != B200_TYPE_I32 || b->ne[0] < a->ne[2] || !is_contiguous(b)) return no("rope: positions must be I32 [n_tokens]");
            const int mode = op->op_params[2];
            if (mode != 0 && mode != 2) return no("rope: only NORMAL and NEOX modes");
            if (op->op_params[15] != 0) return no("rope: channel offset is not supported");
            if (op->src[2] && (op->src[2]->type != B200_TYPE_F32 || op->src[2]->ne[0] < a->ne[0] / 2)) return no("rope: freq factors");
            return true;
        }
        case GGML_OP_SET_ROWS:
            if (!f32_rows(a) || a->ne[2] != 1 || a->ne[3] != 1) return no("set_rows wants a 2-d F32 source");
            if (!b || b->type != B200_TYPE_I64 || !is_contiguous(b) || b->ne[0] != a->ne[1] || b->ne[1] * b->ne[2] != 1) return no("set_rows wants I64 [n_rows] indices");
            if (op->type != B200_TYPE_F16 || op->nb[0] != 2 || op->nb[1] % 2 || op->ne[0] != a->ne[0] || op->ne[2] != 1 || op->ne[3] != 1)
                return no("set_rows wants a 2-d F16 destination");
            return true;
        case GGML_OP_GET_ROWS:
            if (!a || !b || b->type != B200_TYPE_I32 || !is_contiguous(b) || b->ne[1] * b->ne[2] * b->ne[3] != 1) return no("get_rows wants I32 [n] ids");
            if (a->ne[2] != 1 || a->ne[3] != 1 || !f32_rows(op) || op->ne[0] != a->ne[0] || op->ne[1] != b->ne[0]) return no("get_rows: shape");
            if (is_quant_type(a->type)) return is_tiled_tensor(a) && is_contiguous(a) ? true : no("get_rows: quantized table must be a whole tensor");
            if ((a->type == B200_TYPE_F32 && a->nb[0] == 4 && a->nb[1] % 4 == 0) || (a->type == B200_TYPE_F16 && a->nb[0] == 2 && a->nb[1] % 2 == 0)) return true;
            return no("get_rows: table type");
        case GGML_OP_ARGMAX:
            if (!f32_rows(a) || op->type != B200_TYPE_I32 || !is_contiguous(op) || op->ne[0] != nrows_of(a)) return no("argmax wants dense F32 rows");
            return true;
        default: return no("op is outside the quantized mat-mul / flash-attention path");
    }
}

static bool dense_f32(const ggml_tensor *t) { return t && t->type == B200_TYPE_F32 && is_contiguous(t); }
static bool supports_tp(const ggml_tensor *op, std::string *why) {
    auto no = [&](const char *m) { if (why) *why = m; return false; };
    const ggml_tensor *a = op->src[0];
    if (!dense_f32(a) || !dense_f32(op)) return no("tensor-parallel collectives want dense F32 tensors");
    if (op->op == B200_OP_TP_ALL_REDUCE) return op->data == a->data && same_shape(a, op) ? true : no("all-reduce node must alias its source");
    if (a->ne[2] != 1 || a->ne[3] != 1 || op->ne[1] != a->ne[1] || op->ne[0] % a->ne[0] || op->ne[0] / a->ne[0] < 2) return no("all-gather: shape");
    if (op->src[1] && (!dense_f32(op->src[1]) || ggml_nbytes(op->src[1]) < ggml_nbytes(op))) return no("all-gather: scratch tensor too small");
    return true;
}

static bool op_supported(const ggml_tensor *op, std::string *why) {
    switch (op->op) {
        case B200_OP_TP_ALL_REDUCE: case B200_OP_TP_ALL_GATHER: return supports_tp(op, why);
        case GGML_OP_NONE: case GGML_OP_RESHAPE: case GGML_OP_VIEW: case GGML_OP_PERMUTE: case GGML_OP_TRANSPOSE:
            return true;
        case GGML_OP_MUL_MAT: case GGML_OP_MUL_MAT_ID: return supports_mul_mat(op, why);
        case GGML_OP_FLASH_ATTN_EXT: return supports_flash(op, why);
        default: return supports_glue(op, why);
    }
}

// ---- graph_compute ----------------------------------------------------------------------------------
static bool ranges_overlap(const void *a, size_t an, const void *b, size_t bn) {
    const uintptr_t a0 = (uintptr_t)a, b0 = (uintptr_t)b;
    return a0 < b0 + bn && b0 < a0 + an;
}

static int quantized_acts(BackendCtx *bc, const float *x, int64_t ldx, int64_t m, int64_t k, int kind);
static bool fuses_mul_mat_add(const ggml_tensor *mm, const ggml_tensor *add);

// MUL_MAT over one 2-d slice; consecutive mat-muls that read the same rows with the same quantizer
// (q, k, v of a layer; gate and up of an FFN) share one quantization pass.
static int mul_mat_2d(BackendCtx *bc, const ggml_tensor *w, const float *x, int64_t ldx, int64_t m, float *dst, int64_t lddst,
                      const float *addend = nullptr, float *sum = nullptr) {
    const int64_t k = w->ne[0], n = w->ne[1];
    const int route = pick_route(w->type, n, m);
    const int kind = act_kind_for(w->type, route, m);
    if (bc->act_src && ranges_overlap(dst, (size_t)lddst * m * 4, bc->act_src, (size_t)bc->act_ld * bc->act_m * 4)) bc->act_src = nullptr;
    int rc = quantized_acts(bc, x, ldx, m, k, kind);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (sum) return b200_mul_mat_q8_add(w->type, n, k, w->data, bc->act, kind, dst, addend, sum, route, bc->stream);
    return b200_mul_mat_q8(w->type, n, k, m, w->data, bc->act, kind, dst, lddst, route, bc->stream);
}

// the quantized copy of activation rows x in bc->act, made now unless the previous mat-mul left the same one
static int quantized_acts(BackendCtx *bc, const float *x, int64_t ldx, int64_t m, int64_t k, int kind) {
    if (!(bc->act_src == x && bc->act_m == m && bc->act_k == k && bc->act_ld == ldx && bc->act_kind == kind)) {
        const size_t need = b200_act_scratch_nbytes(m, k);
        if (need > bc->act_bytes) {
            if (bc->act) B200_CUDA(cudaFree(bc->act));
            bc->act = nullptr;
            bc->act_bytes = 0;
            B200_CUDA(cudaMalloc(&bc->act, need));
            bc->act_bytes = need;
            bc->generation++;
        }
        bc->act_src = nullptr;
        int rc = b200_quantize_activations_device(kind, m, k, x, ldx, bc->act, bc->stream);
        if (rc != B200_STATUS_SUCCESS) return rc;
        bc->act_src = x; bc->act_m = m; bc->act_k = k; bc->act_ld = ldx; bc->act_kind = kind;
    }
    return B200_STATUS_SUCCESS;
}

// Sibling mat-muls: at one token the k, v and q projections of a layer (and the gate and up projections of its
// FFN) read the same normed row, each through a launch of a few microseconds.  From a one-row Q4_K mat-mul at
// node i, looks a few nodes ahead for other one-row Q4_K mat-muls over the same activation tensor that may run
// early: no node in between touches the sibling's result memory (graph allocators recycle it) or rewrites the
// activations, and the sibling is not itself waiting to be fused with a residual ADD.  Returns how many were
// found (at most 2), their node indices in sib[].
static bool multi_candidate(const ggml_tensor *mm) {
    const ggml_tensor *w = mm->src[0], *x = mm->src[1];
    return mm->op == GGML_OP_MUL_MAT && w && x && w->type == B200_TYPE_Q4_K && w->ne[2] == 1 && w->ne[3] == 1 && w->ne[1] % 8 == 0 &&
           x->ne[1] == 1 && x->ne[2] == 1 && x->ne[3] == 1 && mm->data && supports_mul_mat(mm, nullptr);
}
// the same for a prompt batch or a batched decode step: Q4_K matrices on the 8x8 route over 64 or more activation rows, or 8 to 31
// of them, a multiple of 4 (no tail rows)
static bool multi_candidate_rows(const ggml_tensor *mm) {
    const ggml_tensor *w = mm->src[0], *x = mm->src[1];
    return mm->op == GGML_OP_MUL_MAT && w && x && w->type == B200_TYPE_Q4_K && w->ne[2] == 1 && w->ne[3] == 1 && w->ne[1] % 8 == 0 &&
           (x->ne[1] >= 64 || (x->ne[1] >= 8 && x->ne[1] < 32)) && x->ne[1] % 4 == 0 && x->ne[2] == 1 && x->ne[3] == 1 && mm->data && supports_mul_mat(mm, nullptr);
}
static int find_sibling_mat_muls(const ggml_cgraph *g, int i, int *sib, bool rows = false) {
    const ggml_tensor *first = g->nodes[i];
    const auto cand = [rows](const ggml_tensor *t) { return rows ? multi_candidate_rows(t) : multi_candidate(t); };
    if (!cand(first)) return 0;
    const ggml_tensor *x = first->src[1];
    int found = 0;
    for (int j = i + 1; j < g->n_nodes && j <= i + 12 && found < 2; j++) {
        const ggml_tensor *t = g->nodes[j];
        if (!t) break;
        const bool alias = t->op == GGML_OP_NONE || t->op == GGML_OP_RESHAPE || t->op == GGML_OP_VIEW || t->op == GGML_OP_PERMUTE ||
                           t->op == GGML_OP_TRANSPOSE;
        if (!alias && t->data && ranges_overlap(t->data, ggml_nbytes(t), x->data, ggml_nbytes(x))) break;   // the activations change here
        if (alias || !cand(t) || t->src[1] != x) continue;
        const ggml_tensor *after = j + 1 < g->n_nodes ? g->nodes[j + 1] : nullptr;
        if (after && fuses_mul_mat_add(t, after)) continue;
        if (ranges_overlap(t->data, ggml_nbytes(t), first->data, ggml_nbytes(first))) continue;
        bool free_to_move = true;
        for (int b = i + 1; b < j && free_to_move; b++) {
            const ggml_tensor *mid = g->nodes[b];
            if (!mid) continue;
            if (mid->data && ranges_overlap(mid->data, ggml_nbytes(mid), t->data, ggml_nbytes(t))) free_to_move = false;
            for (int s = 0; s < GGML_MAX_SRC && free_to_move; s++)
                if (mid->src[s] && mid->src[s]->data && ranges_overlap(mid->src[s]->data, ggml_nbytes(mid->src[s]), t->data, ggml_nbytes(t)))
                    free_to_move = false;
        }
        for (int e = 0; e < found && free_to_move; e++)
            if (ranges_overlap(g->nodes[sib[e]]->data, ggml_nbytes(g->nodes[sib[e]]), t->data, ggml_nbytes(t))) free_to_move = false;
        if (free_to_move) sib[found++] = j;
    }
    return found;
}
static int compute_mul_mat_multi(BackendCtx *bc, const ggml_cgraph *g, int i, const int *sib, int n_sib) {
    const ggml_tensor *x = g->nodes[i]->src[1];
    const int64_t k = x->ne[0];
    const int kind = act_kind_for(B200_TYPE_Q4_K, B200_ROUTE_REPACK, 1);
    int64_t n[3];
    const void *w[3];
    float *dst[3];
    for (int e = 0; e <= n_sib; e++) {
        const ggml_tensor *mm = g->nodes[e == 0 ? i : sib[e - 1]];
        n[e] = mm->src[0]->ne[1];
        w[e] = mm->src[0]->data;
        dst[e] = (float *)mm->data;
        if (bc->act_src && ranges_overlap(mm->data, ggml_nbytes(mm), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4)) bc->act_src = nullptr;
    }
    int rc = quantized_acts(bc, (const float *)x->data, (int64_t)(x->nb[1] / 4), 1, k, kind);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return b200_mul_mat_q8_multi(B200_TYPE_Q4_K, k, n_sib + 1, n, w, bc->act, kind, dst, bc->stream);
}

// the same for a prompt batch: one quantization of the activation rows, one call for the sibling matrices
static int compute_mul_mat_multi_rows(BackendCtx *bc, const ggml_cgraph *g, int i, const int *sib, int n_sib) {
    const ggml_tensor *x = g->nodes[i]->src[1];
    const int64_t k = x->ne[0], m = x->ne[1];
    const int kind = act_kind_for(B200_TYPE_Q4_K, B200_ROUTE_REPACK, m);
    int64_t n[3], ld[3];
    const void *w[3];
    float *dst[3];
    for (int e = 0; e <= n_sib; e++) {
        const ggml_tensor *mm = g->nodes[e == 0 ? i : sib[e - 1]];
        n[e] = mm->src[0]->ne[1];
        w[e] = mm->src[0]->data;
        dst[e] = (float *)mm->data;
        ld[e] = (int64_t)(mm->nb[1] / 4);
        if (bc->act_src && ranges_overlap(mm->data, ggml_nbytes(mm), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4)) bc->act_src = nullptr;
    }
    int rc = quantized_acts(bc, (const float *)x->data, (int64_t)(x->nb[1] / 4), m, k, kind);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return b200_mul_mat_q8_rows_multi(B200_TYPE_Q4_K, k, m, n_sib + 1, n, w, bc->act, kind, dst, ld, bc->stream);
}

// fused: a one-row mat-mul whose result the next node adds to a tensor of the same shape (the residual)
static bool fuses_mul_mat_add(const ggml_tensor *mm, const ggml_tensor *add) {
    if (add->op != GGML_OP_ADD || !supports_glue(add, nullptr) || mm->ne[1] != 1 || mm->ne[2] != 1 || mm->ne[3] != 1) return false;
    const ggml_tensor *other = add->src[0] == mm ? add->src[1] : add->src[1] == mm ? add->src[0] : nullptr;
    if (!other || other == mm || !same_shape(other, mm)) return false;
    // the sum must not land on the mat-mul's activations or weights
    return add->data != mm->src[1]->data && add->data != mm->data;
}
// the same for the 8 to 31 rows of a batched decode step, where the few-rows kernels add as they store
static bool fuses_mul_mat_rows_add(const ggml_tensor *mm, const ggml_tensor *add) {
    if (add->op != GGML_OP_ADD || !supports_glue(add, nullptr) || mm->ne[1] < 8 || mm->ne[1] >= 32 || mm->ne[2] != 1 || mm->ne[3] != 1) return false;
    const ggml_tensor *w = mm->src[0], *x = mm->src[1];
    if (!w || !x || w->ne[2] != 1 || w->ne[3] != 1 || x->ne[2] != 1 || x->ne[3] != 1 || !mm->data || !supports_mul_mat(mm, nullptr)) return false;
    const ggml_tensor *other = add->src[0] == mm ? add->src[1] : add->src[1] == mm ? add->src[0] : nullptr;
    if (!other || other == mm || !same_shape(other, mm) || !other->data || !add->data) return false;
    if (mm->nb[0] != 4 || other->nb[0] != 4 || add->nb[0] != 4 || other->type != B200_TYPE_F32 || add->type != B200_TYPE_F32) return false;
    if (!b200_mul_mat_q8_rows_add_fusable(w->type, w->ne[1], mm->ne[1])) return false;
    // the sum must not land on the mat-mul's result, activations or weights
    return !ranges_overlap(add->data, ggml_nbytes(add), mm->data, ggml_nbytes(mm)) && !ranges_overlap(add->data, ggml_nbytes(add), x->data, ggml_nbytes(x)) &&
           !ranges_overlap(add->data, ggml_nbytes(add), w->data, ggml_nbytes(w));
}
static int compute_mul_mat_rows_add(BackendCtx *bc, const ggml_tensor *op, const ggml_tensor *add) {
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    const ggml_tensor *other = add->src[0] == op ? add->src[1] : add->src[0];
    const int64_t k = w->ne[0], n = w->ne[1], m = x->ne[1];
    const int kind = act_kind_for(w->type, pick_route(w->type, n, m), m);
    if (bc->act_src && ranges_overlap(op->data, ggml_nbytes(op), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4)) bc->act_src = nullptr;
    int rc = quantized_acts(bc, (const float *)x->data, (int64_t)(x->nb[1] / 4), m, k, kind);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return b200_mul_mat_q8_rows_add(w->type, n, k, m, w->data, bc->act, kind, (float *)op->data, (int64_t)(op->nb[1] / 4), (const float *)other->data,
                                    (int64_t)(other->nb[1] / 4), (float *)add->data, (int64_t)(add->nb[1] / 4), bc->stream);
}
static int compute_mul_mat_add(BackendCtx *bc, const ggml_tensor *op, const ggml_tensor *add) {
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    const ggml_tensor *other = add->src[0] == op ? add->src[1] : add->src[0];
    return mul_mat_2d(bc, w, (const float *)x->data, (int64_t)(x->nb[1] / 4), 1, (float *)op->data, (int64_t)(op->nb[1] / 4),
                      (const float *)other->data, (float *)add->data);
}

static int compute_mul_mat(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *w = op->src[0], *x = op->src[1];
    for (int64_t i3 = 0; i3 < x->ne[3]; i3++)
        for (int64_t i2 = 0; i2 < x->ne[2]; i2++) {
            const float *xp = (const float *)((const uint8_t *)x->data + i2 * x->nb[2] + i3 * x->nb[3]);
            float *dp = (float *)((uint8_t *)op->data + i2 * op->nb[2] + i3 * op->nb[3]);
            int rc = mul_mat_2d(bc, w, xp, (int64_t)(x->nb[1] / 4), x->ne[1], dp, (int64_t)(op->nb[1] / 4));
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

static float param_f32(const ggml_tensor *op, int i) {
    float f;
    memcpy(&f, &op->op_params[i], 4);
    return f;
}

// The Q8_K kind the first mat-mul among the nodes after `from` that reads t as its activations will ask
// for (0: none, or not a Q8_K kind, or t is not a plain 2-d row block).  The producer of t then quantizes
// it on the way out and the mat-mul finds the quantized copy in place.
static int upcoming_q8_K_kind(const ggml_cgraph *g, int from, const ggml_tensor *t) {
    if (t->ne[2] != 1 || t->ne[3] != 1 || t->ne[0] % GROUP_K || t->nb[1] % 4 || t->ne[1] > 65535) return 0;
    for (int j = from + 1; j < g->n_nodes && j <= from + 24; j++) {
        const ggml_tensor *n = g->nodes[j];
        if (!n || n->op != GGML_OP_MUL_MAT || n->src[1] != t) continue;
        if (!supports_mul_mat(n, nullptr)) return 0;
        const ggml_tensor *w = n->src[0];
        const int kind = act_kind_for(w->type, pick_route(w->type, w->ne[1], t->ne[1]), t->ne[1]);
        return kind == B200_ACT_Q8_K || kind == B200_ACT_Q8_K_4X8 || kind == B200_ACT_Q8_K_MIXED ? kind : 0;
    }
    return 0;
}
static int act_reserve(BackendCtx *bc, int64_t m, int64_t k) {
    const size_t need = b200_act_scratch_nbytes(m, k);
    if (need > bc->act_bytes) {
        B200_CUDA(cudaStreamSynchronize(bc->stream));
        if (bc->act) B200_CUDA(cudaFree(bc->act));
        bc->act = nullptr;
        bc->act_bytes = 0;
        bc->act_src = nullptr;
        B200_CUDA(cudaMalloc(&bc->act, need));
        bc->act_bytes = need;
        bc->generation++;
    }
    return B200_STATUS_SUCCESS;
}
static void act_holds(BackendCtx *bc, const ggml_tensor *t, int kind) {
    bc->act_src = t->data; bc->act_m = t->ne[1]; bc->act_k = t->ne[0]; bc->act_ld = (int64_t)(t->nb[1] / 4); bc->act_kind = kind;
}

// fused: when the node after an RMS_NORM multiplies it by a one-row weight, one kernel writes both; q8_kind != 0:
// it also quantizes the last of them for the mat-muls to come
static int compute_rms_norm(BackendCtx *bc, const ggml_tensor *op, const ggml_tensor *mul, int q8_kind) {
    const ggml_tensor *x = op->src[0];
    const float *w = mul ? (const float *)mul->src[1]->data : nullptr;
    if (q8_kind) {
        const ggml_tensor *last = mul ? mul : op;
        int rc = act_reserve(bc, last->ne[1], last->ne[0]);
        if (rc != B200_STATUS_SUCCESS) return rc;
        bc->act_src = nullptr;
        rc = b200_rms_norm_q8((const float *)x->data, (int64_t)(x->nb[1] / 4), (float *)op->data, (int64_t)(op->nb[1] / 4), w,
                              mul ? (float *)mul->data : nullptr, mul ? (int64_t)(mul->nb[1] / 4) : 0, x->ne[0], nrows_of(x),
                              param_f32(op, 0), bc->act, q8_kind, bc->stream);
        if (rc == B200_STATUS_SUCCESS) act_holds(bc, last, q8_kind);
        return rc;
    }
    return b200_rms_norm((const float *)x->data, (int64_t)(x->nb[1] / 4), (float *)op->data, (int64_t)(op->nb[1] / 4), w,
                         mul ? (float *)mul->data : nullptr, mul ? (int64_t)(mul->nb[1] / 4) : 0, x->ne[0], nrows_of(x),
                         param_f32(op, 0), bc->stream);
}
static bool fuses_norm_mul(const ggml_tensor *norm, const ggml_tensor *mul) {
    return mul->op == GGML_OP_MUL && mul->src[0] == norm && supports_glue(mul, nullptr) && mul->src[1]->ne[0] == norm->ne[0] &&
           nrows_of(mul->src[1]) == 1 && mul->src[1]->data != norm->data;
}
static int compute_binary(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *a = op->src[0], *b = op->src[1];
    return b200_binary(op->op == GGML_OP_ADD ? 0 : 1, (const float *)a->data, (int64_t)(a->nb[1] / 4), (const float *)b->data,
                       (int64_t)(b->nb[1] / 4), b->ne[0], nrows_of(b), (float *)op->data, (int64_t)(op->nb[1] / 4), a->ne[0],
                       nrows_of(a), bc->stream);
}
// fused: when the node after a SILU multiplies it by a tensor of the same shape, one kernel writes both
static int compute_silu(BackendCtx *bc, const ggml_tensor *op, const ggml_tensor *mul, int q8_kind) {
    const ggml_tensor *x = op->src[0];
    const ggml_tensor *g = mul ? mul->src[1] : nullptr;
    if (q8_kind) {
        const ggml_tensor *last = mul ? mul : op;
        int rc = act_reserve(bc, last->ne[1], last->ne[0]);
        if (rc != B200_STATUS_SUCCESS) return rc;
        bc->act_src = nullptr;
        rc = b200_silu_q8((const float *)x->data, (int64_t)(x->nb[1] / 4), g ? (const float *)g->data : nullptr,
                          g ? (int64_t)(g->nb[1] / 4) : 0, (float *)op->data, (int64_t)(op->nb[1] / 4), mul ? (float *)mul->data : nullptr,
                          mul ? (int64_t)(mul->nb[1] / 4) : 0, x->ne[0], nrows_of(x), bc->silu_wide, bc->act, q8_kind, bc->stream);
        if (rc == B200_STATUS_SUCCESS) act_holds(bc, last, q8_kind);
        return rc;
    }
    return b200_silu((const float *)x->data, (int64_t)(x->nb[1] / 4), g ? (const float *)g->data : nullptr,
                     g ? (int64_t)(g->nb[1] / 4) : 0, (float *)op->data, (int64_t)(op->nb[1] / 4), mul ? (float *)mul->data : nullptr,
                     mul ? (int64_t)(mul->nb[1] / 4) : 0, x->ne[0], nrows_of(x), bc->silu_wide, bc->stream);
}
static bool fuses_silu_mul(const ggml_tensor *silu, const ggml_tensor *mul) {
    return mul->op == GGML_OP_MUL && mul->src[0] == silu && supports_glue(mul, nullptr) && same_shape(mul->src[1], silu);
}

// The host's view of a ROPE node's positions: the copy set_tensor kept, else a read-back (which makes the
// node list uncapturable: issuing it talks to the device).
static int rope_positions(BackendCtx *bc, const ggml_tensor *op, std::vector<int32_t> *p) {
    const ggml_tensor *pos = op->src[1];
    const int64_t n_tok = op->src[0]->ne[2];
    p->clear();
    if (in_our_buffer(pos)) {
        BufferCtx *c = bctx(pos->buffer);
        std::lock_guard<std::mutex> lk(c->mu);
        auto it = c->i32_shadow.find(pos->data);
        if (it != c->i32_shadow.end() && (int64_t)it->second.size() >= n_tok) p->assign(it->second.begin(), it->second.begin() + n_tok);
    }
    if (p->empty() && n_tok > 0) {
        bc->capturable = false;
        p->resize(n_tok);
        B200_CUDA(cudaStreamSynchronize(bc->stream));
        B200_CUDA(cudaMemcpy(p->data(), pos->data, n_tok * 4, cudaMemcpyDeviceToHost));
    }
    return B200_STATUS_SUCCESS;
}
static int rope_factors(BackendCtx *bc, const ggml_tensor *op, std::vector<float> *f) {
    const ggml_tensor *ff = op->src[2];
    f->clear();
    if (!ff) return B200_STATUS_SUCCESS;
    bc->capturable = false;
    f->resize(op->src[0]->ne[0] / 2);
    B200_CUDA(cudaStreamSynchronize(bc->stream));
    B200_CUDA(cudaMemcpy(f->data(), ff->data, f->size() * 4, cudaMemcpyDeviceToHost));
    return B200_STATUS_SUCCESS;
}
static std::vector<int32_t> rope_param_key(const ggml_tensor *op, const std::vector<float> &factors) {
    std::vector<int32_t> key(op->op_params, op->op_params + 16);
    key.push_back((int32_t)op->src[0]->ne[0]);
    for (float f : factors) { int32_t b; memcpy(&b, &f, 4); key.push_back(b); }
    return key;
}
static int rope_fill_host(BackendCtx *bc, const ggml_tensor *op, const int32_t *pos, int64_t rows, const std::vector<float> &factors) {
    bc->rope_host.resize((size_t)rows * op->src[0]->ne[0]);
    return b200_rope_table(pos, rows, op->src[0]->ne[0], factors.empty() ? nullptr : factors.data(), op->op_params[1], op->op_params[4],
                           param_f32(op, 5), param_f32(op, 6), param_f32(op, 7), param_f32(op, 8), param_f32(op, 9), param_f32(op, 10),
                           bc->rope_host.data());
}

// Before a node list is issued: every ROPE node's by-position table exists and reaches its largest
// position.  All device work this needs (allocation, upload) happens here, outside any capture.
static int rope_prepare(BackendCtx *bc, const ggml_tensor *op) {
    std::vector<int32_t> p;
    std::vector<float> factors;
    int rc = rope_positions(bc, op, &p);
    if (rc == B200_STATUS_SUCCESS) rc = rope_factors(bc, op, &factors);
    if (rc != B200_STATUS_SUCCESS || p.empty()) return rc;
    const int32_t pmin = *std::min_element(p.begin(), p.end()), pmax = *std::max_element(p.begin(), p.end());
    if (pmin < 0 || pmax >= ROPE_TABLE_MAX_ROWS) {
        bc->capturable = false;   // served by the per-token table, built while the node is issued
        return B200_STATUS_SUCCESS;
    }
    const std::vector<int32_t> key = rope_param_key(op, factors);
    BackendCtx::RopeTable *t = nullptr;
    for (auto &cand : bc->rope_by_pos)
        if (cand.key == key) t = &cand;
    if (t && pmax < t->rows) {
        t->used = ++bc->rope_clock;
        return B200_STATUS_SUCCESS;
    }
    if (!t) {
        if (bc->rope_by_pos.size() >= ROPE_TABLES_KEPT) {
            auto lru = std::min_element(bc->rope_by_pos.begin(), bc->rope_by_pos.end(),
                                        [](const BackendCtx::RopeTable &a, const BackendCtx::RopeTable &b) { return a.used < b.used; });
            B200_CUDA(cudaStreamSynchronize(bc->stream));
            if (lru->dev) B200_CUDA(cudaFree(lru->dev));
            bc->rope_by_pos.erase(lru);
            bc->generation++;
        }
        bc->rope_by_pos.emplace_back();
        t = &bc->rope_by_pos.back();
        t->key = key;
    }
    int64_t rows = ROPE_TABLE_MIN_ROWS;
    while (rows <= pmax) rows *= 2;
    std::vector<int32_t> all(rows);
    for (int64_t i = 0; i < rows; i++) all[i] = (int32_t)i;
    rc = rope_fill_host(bc, op, all.data(), rows, factors);
    if (rc != B200_STATUS_SUCCESS) return rc;
    B200_CUDA(cudaStreamSynchronize(bc->stream));   // launches in flight may still read the smaller table
    if (t->dev) B200_CUDA(cudaFree(t->dev));
    t->dev = nullptr;
    t->rows = 0;
    bc->generation++;
    B200_CUDA(cudaMalloc((void **)&t->dev, bc->rope_host.size() * 4));
    B200_CUDA(cudaMemcpy(t->dev, bc->rope_host.data(), bc->rope_host.size() * 4, cudaMemcpyHostToDevice));
    t->rows = rows;
    t->used = ++bc->rope_clock;
    return B200_STATUS_SUCCESS;
}

static int compute_rope(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *x = op->src[0], *pos = op->src[1];
    const int64_t ne0 = x->ne[0], n_head = x->ne[1], n_tok = x->ne[2];
    if (n_tok == 0 || n_head == 0) return B200_STATUS_SUCCESS;
    if (!op->src[2]) {
        const std::vector<int32_t> key = rope_param_key(op, std::vector<float>());
        for (auto &t : bc->rope_by_pos)
            if (t.key == key && t.dev)   // rope_prepare made it cover this node's positions; the kernel checks again
                return b200_rope((const float *)x->data, (int64_t)x->nb[1], (int64_t)x->nb[2], (float *)op->data, (int64_t)op->nb[1],
                                 (int64_t)op->nb[2], t.dev, (const int32_t *)pos->data, t.rows, ne0, n_head, n_tok, op->op_params[1],
                                 op->op_params[2], bc->stream);
    }
    // per-token table: frequency factors, or positions a by-position table cannot hold
    std::vector<int32_t> p;
    std::vector<float> factors;
    int rc = rope_positions(bc, op, &p);
    if (rc == B200_STATUS_SUCCESS) rc = rope_factors(bc, op, &factors);
    if (rc != B200_STATUS_SUCCESS) return rc;
    bc->capturable = false;
    if (!factors.empty()) {
        const std::vector<int32_t> key = rope_param_key(op, factors);
        for (auto &t : bc->rope_by_pos)
            if (t.key == key && t.dev && *std::min_element(p.begin(), p.end()) >= 0 && *std::max_element(p.begin(), p.end()) < t.rows)
                return b200_rope((const float *)x->data, (int64_t)x->nb[1], (int64_t)x->nb[2], (float *)op->data, (int64_t)op->nb[1],
                                 (int64_t)op->nb[2], t.dev, (const int32_t *)pos->data, t.rows, ne0, n_head, n_tok, op->op_params[1],
                                 op->op_params[2], bc->stream);
    }
    std::vector<int32_t> key = rope_param_key(op, factors);
    key.insert(key.end(), p.begin(), p.end());
    const size_t floats = (size_t)n_tok * ne0;
    if (key != bc->rope_key || bc->rope_dev == nullptr) {
        bc->rope_key.clear();
        if (floats > bc->rope_dev_floats) {
            B200_CUDA(cudaStreamSynchronize(bc->stream));
            if (bc->rope_dev) B200_CUDA(cudaFree(bc->rope_dev));
            bc->rope_dev = nullptr;
            bc->rope_dev_floats = 0;
            B200_CUDA(cudaMalloc((void **)&bc->rope_dev, floats * 4));
            bc->rope_dev_floats = floats;
        }
        rc = rope_fill_host(bc, op, p.data(), n_tok, factors);
        if (rc != B200_STATUS_SUCCESS) return rc;
        // pageable source: the runtime has taken its copy of rope_host when this returns
        B200_CUDA(cudaMemcpyAsync(bc->rope_dev, bc->rope_host.data(), floats * 4, cudaMemcpyHostToDevice, bc->stream));
        bc->rope_key = key;
    }
    return b200_rope((const float *)x->data, (int64_t)x->nb[1], (int64_t)x->nb[2], (float *)op->data, (int64_t)op->nb[1],
                     (int64_t)op->nb[2], bc->rope_dev, nullptr, 0, ne0, n_head, n_tok, op->op_params[1], op->op_params[2], bc->stream);
}

static int compute_set_rows(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *x = op->src[0], *idx = op->src[1];
    return b200_set_rows_f16((const float *)x->data, (int64_t)(x->nb[1] / 4), (const int64_t *)idx->data, op->data,
                             (int64_t)(op->nb[1] / 2), op->ne[1], x->ne[0], x->ne[1], bc->stream);
}
// ---- ROPE / SET_ROWS nodes that share a launch (glue_batch_kernel) ------------------------------------------
static bool is_alias_op(const ggml_tensor *t) {
    return t->op == GGML_OP_NONE || t->op == GGML_OP_RESHAPE || t->op == GGML_OP_VIEW || t->op == GGML_OP_PERMUTE || t->op == GGML_OP_TRANSPOSE;
}
// a ROPE served from a by-position table (no frequency factors, positions the table covers: rope_prepare saw to it)
static bool glue_rope_op(BackendCtx *bc, const ggml_tensor *op, GlueOp *o) {
    const ggml_tensor *x = op->src[0], *pos = op->src[1];
    if (op->src[2] || x->ne[0] == 0 || x->ne[1] == 0 || x->ne[2] == 0 || x->ne[3] != 1) return false;
    const int mode = op->op_params[2];
    if (mode != 0 && mode != 2) return false;
    const std::vector<int32_t> key = rope_param_key(op, std::vector<float>());
    for (auto &t : bc->rope_by_pos)
        if (t.key == key && t.dev) {
            *o = GlueOp{};
            o->kind = GLUE_ROPE;
            o->ne0 = (int)x->ne[0];
            o->n_head = (int)x->ne[1];
            o->n_dims = op->op_params[1];
            o->neox = mode == 2;
            o->total = x->ne[2] * x->ne[1] * (x->ne[0] / 2);
            o->x = (const float *)x->data;
            o->x_nb1 = (int64_t)x->nb[1];
            o->x_nb2 = (int64_t)x->nb[2];
            o->y = (float *)op->data;
            o->y_nb1 = (int64_t)op->nb[1];
            o->y_nb2 = (int64_t)op->nb[2];
            o->table = t.dev;
            o->rows = (const int32_t *)pos->data;
            o->n_rows = t.rows;
            return true;
        }
    return false;
}
static void glue_set_rows_op(const ggml_tensor *op, GlueOp *o) {
    const ggml_tensor *x = op->src[0], *idx = op->src[1];
    *o = GlueOp{};
    o->kind = GLUE_SET_ROWS;
    o->ne0 = (int)x->ne[0];
    o->total = x->ne[0] * x->ne[1];
    o->x = (const float *)x->data;
    o->x_nb1 = (int64_t)(x->nb[1] / 4);
    o->cache = op->data;
    o->cache_stride = (int64_t)(op->nb[1] / 2);
    o->cache_rows = op->ne[1];
    o->cache_idx = (const int64_t *)idx->data;
}
// From node i (a ROPE or a SET_ROWS) on, the nodes that can run in one launch: ROPEs served from a table,
// SET_ROWS that read one of those ROPEs' whole result (they ride with it) or something the batch does not write,
// none of them reading or overwriting what an earlier member writes.  members[] = the node indices taken.
struct TensorRange {
    const void *p;
    size_t n;
};
static int gather_glue_batch(BackendCtx *bc, const ggml_cgraph *g, int i, const std::vector<char> &done, GlueBatch *b, int *members) {
    b->count = 0;
    int n_members = 0;
    std::vector<TensorRange> ins, outs;
    const ggml_tensor *rope_node[GLUE_BATCH_MAX] = {nullptr, nullptr, nullptr, nullptr};
    for (int j = i; j < g->n_nodes && n_members < 2 * GLUE_BATCH_MAX; j++) {
        const ggml_tensor *t = g->nodes[j];
        if (!t) break;
        if (done[j] || is_alias_op(t)) continue;
        if ((t->op != GGML_OP_ROPE && t->op != GGML_OP_SET_ROWS) || !op_supported(t, nullptr) || !t->data) break;
        std::vector<TensorRange> t_in, t_out;
        for (int s = 0; s < GGML_MAX_SRC; s++)
            if (t->src[s] && t->src[s]->data) t_in.push_back({t->src[s]->data, ggml_nbytes(t->src[s])});
        t_out.push_back({t->data, ggml_nbytes(t)});
        int ride = -1;   // a SET_ROWS that takes a member ROPE's result as it is made
        if (t->op == GGML_OP_SET_ROWS) {
            const ggml_tensor *x = t->src[0];
            for (int e = 0; e < b->count; e++) {
                const GlueOp &r = b->op[e];
                if (r.kind == GLUE_ROPE && !r.cache && rope_node[e] && x->data == rope_node[e]->data && x->ne[0] == (int64_t)r.ne0 * r.n_head &&
                    (int64_t)x->nb[1] == x->ne[0] * 4 && r.y_nb1 == (int64_t)r.ne0 * 4 && r.y_nb2 == x->ne[0] * 4 &&
                    x->ne[1] * x->ne[0] == r.total * 2)
                    ride = e;
            }
        }
        // what this node reads must not be written by the batch (other than the ROPE it rides with), and what it
        // writes must not be read or written by the batch
        bool clash = false;
        for (const TensorRange &a : t_in)
            for (const TensorRange &o : outs)
                if (ranges_overlap(a.p, a.n, o.p, o.n) && !(ride >= 0 && o.p == rope_node[ride]->data)) clash = true;
        for (const TensorRange &a : t_out) {
            for (const TensorRange &o : outs)
                if (ranges_overlap(a.p, a.n, o.p, o.n)) clash = true;
            for (const TensorRange &o : ins)
                if (ranges_overlap(a.p, a.n, o.p, o.n)) clash = true;
        }
        if (clash) break;
        if (ride >= 0) {
            GlueOp s;
            glue_set_rows_op(t, &s);
            b->op[ride].cache = s.cache;
            b->op[ride].cache_stride = s.cache_stride;
            b->op[ride].cache_rows = s.cache_rows;
            b->op[ride].cache_idx = s.cache_idx;
        } else {
            if (b->count == GLUE_BATCH_MAX) break;
            GlueOp o;
            if (t->op == GGML_OP_ROPE) {
                if (!glue_rope_op(bc, t, &o)) break;
                rope_node[b->count] = t;
            } else {
                glue_set_rows_op(t, &o);
            }
            b->op[b->count++] = o;
        }
        ins.insert(ins.end(), t_in.begin(), t_in.end());
        outs.insert(outs.end(), t_out.begin(), t_out.end());
        members[n_members++] = j;
    }
    return n_members;
}

static int compute_get_rows(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *t = op->src[0], *ids = op->src[1];
    if (!is_quant_type(t->type)) {
        // dense tables may be row-strided views: pass the stride through the row length the kernel uses
        const int64_t es = t->type == B200_TYPE_F32 ? 4 : 2;
        B200_REQUIRE((int64_t)t->nb[1] == t->ne[0] * es, "get_rows: dense table rows must be packed");
    }
    return b200_get_rows(t->type, t->data, t->ne[0], t->ne[1], (const int32_t *)ids->data, ids->ne[0], (float *)op->data,
                         (int64_t)(op->nb[1] / 4), bc->stream);
}
static int compute_argmax(BackendCtx *bc, const ggml_tensor *op) {
    const ggml_tensor *x = op->src[0];
    return b200_argmax((const float *)x->data, (int64_t)(x->nb[1] / 4), x->ne[0], nrows_of(x), (int32_t *)op->data, bc->stream);
}

// A SILU whose product with the up projection comes a few nodes later (the graph's depth-first order
// puts the up mat-mul between them: crates/llama/src/graph_arch.rs:1137-1151) waits for that MUL, and one
// kernel then writes both results.  Returns the MUL's index, or -1 when the SILU has to run on its own.
static int find_silu_mul(const ggml_cgraph *g, int i) {
    const ggml_tensor *silu = g->nodes[i];
    for (int j = i + 1; j < g->n_nodes && j <= i + 4; j++) {
        const ggml_tensor *n = g->nodes[j];
        if (!n) return -1;
        if (n->op == GGML_OP_MUL && fuses_silu_mul(silu, n)) return j;
        if (n->view_src == silu) return -1;
        for (int s = 0; s < GGML_MAX_SRC; s++)
            if (n->src[s] == silu) return -1;
        // a node that overwrites the SILU's input or output in place would change what the fused kernel reads
        if (n->data && silu->src[0]->data &&
            (ranges_overlap(n->data, ggml_nbytes(n), silu->src[0]->data, ggml_nbytes(silu->src[0])) ||
             ranges_overlap(n->data, ggml_nbytes(n), silu->data, ggml_nbytes(silu))))
            return -1;
    }
    return -1;
}

// A norm / silu whose result's first reader is the very next non-alias node, a one-row Q4_K mat-mul on the 8x8 gemv
// route: the op and the quantization of its result run inside that mat-mul's kernel (b200_mul_mat_row_fused).
// Returns the mat-mul's node index, or -1.
static int fusable_row_mat_mul(const ggml_cgraph *g, int from, const ggml_tensor *t) {
    if (t->ne[1] != 1 || t->ne[2] != 1 || t->ne[3] != 1 || t->ne[0] % GROUP_K || ((uintptr_t)t->data & 15)) return -1;
    for (int j = from + 1; j < g->n_nodes; j++) {
        const ggml_tensor *n = g->nodes[j];
        if (!n) return -1;
        if (is_alias_op(n)) continue;
        return n->op == GGML_OP_MUL_MAT && n->src[1] == t && multi_candidate(n) ? j : -1;
    }
    return -1;
}
// which prologues ride inside the mat-mul kernels: bit 0 quantization only, bit 1 norm in front of at most two row
// tiles per SM, bit 2 silu, bit 3 norm in front of any number of row tiles (B200_FUSE_PROLOGUE_MASK, read once)
// Measured on the 8B-shape single-token step: only the quantization-only prologue pays (every CTA of the mat-mul
// redoes a norm or silu prologue, and that costs more than the launch it saves), so that is the default.
static int prologue_mask() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_FUSE_PROLOGUE_MASK");
        v = e ? atoi(e) : 1;
    }
    return v;
}
// B200_DEBUG_SKIP: a comma-separated list of node classes whose launches are left out (fa, rms, silu, glue, add,
// getrows, argmax, mm:<rows>x<k>), for measuring what a class of kernels costs inside a replayed step by taking it
// out.  The step's results are meaningless with it; never set outside a measurement.
static bool debug_skip(const ggml_tensor *op) {
    static std::string list = [] { const char *e = getenv("B200_DEBUG_SKIP"); return std::string(e ? e : ""); }();
    if (list.empty()) return false;
    auto has = [&](const std::string &tok) { return ("," + list + ",").find("," + tok + ",") != std::string::npos; };
    switch (op->op) {
        case GGML_OP_FLASH_ATTN_EXT: return has("fa");
        case GGML_OP_RMS_NORM: return has("rms");
        case GGML_OP_UNARY: return has("silu");
        case GGML_OP_ROPE: case GGML_OP_SET_ROWS: return has("glue");
        case GGML_OP_ADD: return has("add");
        case GGML_OP_GET_ROWS: return has("getrows");
        case GGML_OP_ARGMAX: return has("argmax");
        case GGML_OP_MUL_MAT:
            return has("mm:" + std::to_string(op->src[0]->ne[1]) + "x" + std::to_string(op->src[0]->ne[0])) || has("mm");
        default: return false;
    }
}
static int64_t row_tiles_of(const ggml_cgraph *g, int j) {
    // the row tiles a fused launch starting at mat-mul j would span: the mat-mul and the siblings that may join it
    const ggml_tensor *first = g->nodes[j];
    int64_t tiles = (first->src[0]->ne[1] + TILE_ROWS - 1) / TILE_ROWS;
    int sib[2];
    const int n_sib = find_sibling_mat_muls(g, j, sib);
    for (int e = 0; e < n_sib; e++) tiles += (g->nodes[sib[e]]->src[0]->ne[1] + TILE_ROWS - 1) / TILE_ROWS;
    return tiles;
}
struct PendingPrologue {
    bool active = false;
    b200_act_prologue pro;
    const ggml_tensor *act_tensor = nullptr;   // the tensor whose quantized row the mat-mul's kernel leaves in bc->act
};

// One-row Q4_K mat-mul(s) with a prologue: node i and its siblings (or node i and the residual ADD after it).
static int compute_mul_mat_row_fused(BackendCtx *bc, const ggml_cgraph *g, int i, const int *sib, int n_sib, const ggml_tensor *add,
                                     b200_act_prologue pro, const ggml_tensor *act_tensor) {
    const ggml_tensor *first = g->nodes[i];
    const int64_t k = first->src[0]->ne[0];
    int64_t n[3];
    const void *w[3];
    float *dst[3];
    for (int e = 0; e <= n_sib; e++) {
        const ggml_tensor *mm = g->nodes[e == 0 ? i : sib[e - 1]];
        n[e] = mm->src[0]->ne[1];
        w[e] = mm->src[0]->data;
        dst[e] = (float *)mm->data;
    }
    int rc = act_reserve(bc, 1, k);
    if (rc != B200_STATUS_SUCCESS) return rc;
    bc->act_src = nullptr;
    pro.dev_act_out = bc->act;
    const ggml_tensor *other = add ? (add->src[0] == first ? add->src[1] : add->src[0]) : nullptr;
    rc = b200_mul_mat_row_fused(B200_TYPE_Q4_K, k, n_sib + 1, n, w, dst, &pro, other ? (const float *)other->data : nullptr,
                                add ? (float *)add->data : nullptr, bc->stream);
    if (rc == B200_STATUS_SUCCESS) act_holds(bc, act_tensor, B200_ACT_Q8_K);
    return rc;
}

// ---- a one-token step as one persistent kernel ------------------------------------------------------------
// The node list of a single-token llama step (crates/llama/src/graph_arch.rs:106-248 with the flash-attention branch
// of attn_kv_cached, :1173-1240, and build_ffn_silu_par, :1128-1158) is, per layer and with the aliasing nodes
// (RESHAPE / VIEW / PERMUTE) left out, the 20 operations of LAYER_OPS below; after the last layer come the output
// norm, GET_ROWS of the wanted row and the output mat-mul.  When a list has exactly that form, every weight is
// Q4_K or Q6_K in tile layout with whole row tiles, the numerics policy is the tolerant one (attention runs in its
// fast form) and no tensor-parallel group is attached, the nodes from the first layer's norm to the logits run as
// decode_persistent_kernel.  Anything else keeps the node-by-node path.
static const int LAYER_OPS[20] = {GGML_OP_RMS_NORM, GGML_OP_MUL, GGML_OP_MUL_MAT, GGML_OP_ROPE, GGML_OP_SET_ROWS, GGML_OP_MUL_MAT, GGML_OP_SET_ROWS,
                                  GGML_OP_MUL_MAT, GGML_OP_ROPE, GGML_OP_FLASH_ATTN_EXT, GGML_OP_MUL_MAT, GGML_OP_ADD, GGML_OP_RMS_NORM, GGML_OP_MUL,
                                  GGML_OP_MUL_MAT, GGML_OP_UNARY, GGML_OP_MUL_MAT, GGML_OP_MUL, GGML_OP_MUL_MAT, GGML_OP_ADD};

static bool step_weight_ok(const ggml_tensor *mm, const ggml_tensor *acts) {
    const ggml_tensor *w = mm->src[0];
    return supports_mul_mat(mm, nullptr) && mm->src[1] && mm->src[1]->data == acts->data && (w->type == B200_TYPE_Q4_K || w->type == B200_TYPE_Q6_K) &&
           is_tiled_tensor(w) && w->ne[2] == 1 && w->ne[1] % TILE_ROWS == 0 && mm->ne[1] == 1 && mm->ne[2] == 1 && mm->ne[3] == 1 &&
           ((uintptr_t)mm->data & 15) == 0 && ((uintptr_t)acts->data & 15) == 0;
}
static void step_mat(DpMat *m, const ggml_tensor *mm, int epi) {
    memset(m, 0, sizeof(*m));
    m->tiles = (const uint8_t *)mm->src[0]->data;
    m->dst = (float *)mm->data;
    m->type = mm->src[0]->type;
    m->n_tiles = (int)(mm->src[0]->ne[1] / TILE_ROWS);
    m->epi = epi;
}
static const ggml_tensor *other_src(const ggml_tensor *op, const ggml_tensor *one) { return op->src[0] == one ? op->src[1] : op->src[0]; }
static bool norm_pair_ok(const ggml_tensor *norm, const ggml_tensor *mul) {
    return norm->ne[1] == 1 && norm->ne[2] == 1 && norm->ne[3] == 1 && norm->ne[0] % GROUP_K == 0 && fuses_norm_mul(norm, mul) &&
           dense_f32(norm->src[0]) && dense_f32(mul) && ((uintptr_t)norm->src[0]->data & 15) == 0 && ((uintptr_t)mul->src[1]->data & 15) == 0 &&
           ((uintptr_t)norm->data & 15) == 0 && ((uintptr_t)mul->data & 15) == 0;
}

// fills `phases` for the nodes [*first, *last) of g; false: not a step the kernel takes
static bool match_decode_step(BackendCtx *bc, const ggml_cgraph *g, std::vector<DpPhase> *phases, int *first, int *last, int *fa_splits,
                              int *fa_heads) {
    if (!bc->persistent_decode || numerics_mode() != 1 || bc->tp != nullptr) return false;
    std::vector<int> ops;   // the nodes that compute something
    for (int i = 0; i < g->n_nodes; i++)
        if (g->nodes[i] && !is_alias_op(g->nodes[i])) ops.push_back(i);
    auto T = [&](size_t c) { return g->nodes[ops[c]]; };
    size_t c0 = 0;
    while (c0 < ops.size() && T(c0)->op != GGML_OP_RMS_NORM) c0++;
    size_t c = c0;
    int n_layer = 0;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, bc->device) != cudaSuccess || sms <= 0) return false;
    int rot = 0;
    auto gemv_phase = [&](int prologue, const ggml_tensor *x_in, const ggml_tensor *norm, const ggml_tensor *mul, int k) {
        DpPhase P;
        memset(&P, 0, sizeof(P));
        P.kind = DP_GEMV;
        P.prologue = prologue;
        P.k = k;
        P.nb = k / GROUP_K;
        P.x = (const float *)x_in->data;
        if (prologue == DP_PRO_NORM) {
            P.norm_w = (const float *)mul->src[1]->data;
            P.eps = param_f32(norm, 0);
            P.y = (float *)norm->data;
            P.y_mul = (float *)mul->data;
        }
        return P;
    };
    auto close_phase = [&](DpPhase &P) {
        P.jobs = 0;
        if (P.pair) P.jobs = P.mat[0].n_tiles;
        else for (int m = 0; m < P.n_mat; m++) P.jobs += P.mat[m].n_tiles;
        P.rot = rot % sms;
        rot = (rot + P.jobs) % sms;
        phases->push_back(P);
    };
    while (c + 20 <= ops.size()) {
        bool is_layer = true;
        for (int j = 0; j < 20 && is_layer; j++) is_layer = T(c + j)->op == LAYER_OPS[j];
        if (!is_layer) break;
        const ggml_tensor *norm1 = T(c), *mul1 = T(c + 1), *mmk = T(c + 2), *ropek = T(c + 3), *setk = T(c + 4), *mmv = T(c + 5), *setv = T(c + 6);
        const ggml_tensor *mmq = T(c + 7), *ropeq = T(c + 8), *fa = T(c + 9), *mmo = T(c + 10), *add1 = T(c + 11), *norm2 = T(c + 12), *mul2 = T(c + 13);
        const ggml_tensor *mmg = T(c + 14), *silu = T(c + 15), *mmu = T(c + 16), *gmul = T(c + 17), *mmd = T(c + 18), *add2 = T(c + 19);
        if (!norm_pair_ok(norm1, mul1) || !norm_pair_ok(norm2, mul2)) return false;
        if (!step_weight_ok(mmk, mul1) || !step_weight_ok(mmv, mul1) || !step_weight_ok(mmq, mul1)) return false;
        const int64_t E = norm1->ne[0];
        if (mmk->src[0]->ne[0] != E || mmg->src[0]->ne[0] != E) return false;
        // rotation of K and Q: adjacent channel pairs, a by-position table, positions on the device
        const ggml_tensor *ropes[2] = {ropek, ropeq};
        const ggml_tensor *srcs[2] = {mmk, mmq};
        const float *table = nullptr;
        int64_t table_rows = 0;
        for (int r = 0; r < 2; r++) {
            const ggml_tensor *ro = ropes[r];
            if (!supports_glue(ro, nullptr) || ro->src[2] || ro->op_params[2] != 0 || ro->src[0]->data != srcs[r]->data) return false;
            if (ro->src[0]->ne[2] != 1 || ro->ne[0] != 128 || ro->op_params[1] > 128 || ro->op_params[1] % 2) return false;
            if ((int64_t)ro->src[0]->nb[1] != ro->ne[0] * 4 || (int64_t)ro->nb[1] != ro->ne[0] * 4 || !ro->src[1] || ro->src[1]->type != B200_TYPE_I32) return false;
            const std::vector<int32_t> key = rope_param_key(ro, std::vector<float>());
            const float *t = nullptr;
            for (auto &cand : bc->rope_by_pos)
                if (cand.key == key && cand.dev) { t = cand.dev; table_rows = cand.rows; }
            if (!t || (table && t != table)) return false;
            table = t;
        }
        if (ropek->src[1]->data != ropeq->src[1]->data) return false;
        // cache writes: F16 rows of the layer's cache, one cell index for both
        if (setk->src[0]->data != ropek->data || setv->src[0]->data != mmv->data || setk->type != B200_TYPE_F16 || setv->type != B200_TYPE_F16) return false;
        if (!supports_glue(setk, nullptr) || !supports_glue(setv, nullptr) || setk->src[1]->data != setv->src[1]->data || setk->src[1]->type != B200_TYPE_I64) return false;
        if (setk->ne[0] != mmk->ne[0] || setv->ne[0] != mmv->ne[0] || setk->nb[1] != setk->ne[0] * 2 || setv->nb[1] != setv->ne[0] * 2) return false;
        // attention: one token, head size 128, the rotated Q, the caches just written
        if (!supports_flash(fa, nullptr) || fa->src[0]->data != ropeq->data || fa->src[4] || fa->src[0]->ne[0] != 128 || fa->src[2]->ne[0] != 128) return false;
        if (fa->src[0]->ne[1] != 1 || !fa->src[3] || !is_contiguous(fa) || ((uintptr_t)fa->data & 15)) return false;
        if (fa->src[1]->data != setk->data || fa->src[2]->data != setv->data) return false;
        if (param_f32(fa, 1) != 0.0f || param_f32(fa, 2) != 0.0f) return false;
        if (!step_weight_ok(mmo, fa) || !fuses_mul_mat_add(mmo, add1)) return false;
        if (!step_weight_ok(mmg, mul2) || !step_weight_ok(mmu, mul2) || norm2->src[0]->data != add1->data) return false;
        if (silu->src[0] != mmg || !supports_glue(silu, nullptr) || !fuses_silu_mul(silu, gmul) || other_src(gmul, silu) != mmu) return false;
        if (mmg->src[0]->ne[1] != mmu->src[0]->ne[1] || !step_weight_ok(mmd, gmul) || !fuses_mul_mat_add(mmd, add2)) return false;
        if (other_src(add2, mmd)->data != add1->data || other_src(add1, mmo)->data != norm1->src[0]->data) return false;
        if (!dense_f32(add1) || !dense_f32(add2) || !dense_f32(gmul)) return false;

        // phase 1: norm | K, V, Q | rope, cache rows
        DpPhase P1 = gemv_phase(DP_PRO_NORM, norm1->src[0], norm1, mul1, (int)E);
        P1.n_mat = 3;
        step_mat(&P1.mat[0], mmq, DP_EPI_ROPE);
        P1.mat[0].dst_raw = (float *)mmq->data;
        P1.mat[0].dst = (float *)ropeq->data;
        step_mat(&P1.mat[1], mmk, DP_EPI_ROPE_CACHE);
        P1.mat[1].dst_raw = (float *)mmk->data;
        P1.mat[1].dst = (float *)ropek->data;
        P1.mat[1].cache = (__half *)setk->data;
        step_mat(&P1.mat[2], mmv, DP_EPI_CACHE);
        P1.mat[2].cache = (__half *)setv->data;
        P1.head_dim = 128;
        P1.n_dims = ropek->op_params[1];
        P1.rope_table = table;
        P1.rope_rows = table_rows;
        P1.pos = (const int32_t *)ropek->src[1]->data;
        P1.cell = (const int64_t *)setk->src[1]->data;
        P1.cache_stride = setk->ne[0];
        P1.cache_rows = setk->ne[1];
        close_phase(P1);
        // phase 2: attention
        DpPhase P2;
        memset(&P2, 0, sizeof(P2));
        P2.kind = DP_ATTN;
        {
            const ggml_tensor *q = fa->src[0], *k = fa->src[1], *v = fa->src[2], *m = fa->src[3];
            b200_flash_attn_args &a = P2.fa;
            a.dk = q->ne[0]; a.dv = v->ne[0]; a.n_tok = q->ne[1]; a.n_head = q->ne[2]; a.n_head_kv = k->ne[2]; a.n_kv = k->ne[1];
            a.q = (const float *)q->data; a.q_nb1 = (int64_t)q->nb[1]; a.q_nb2 = (int64_t)q->nb[2];
            a.k = k->data; a.k_nb1 = (int64_t)k->nb[1]; a.k_nb2 = (int64_t)k->nb[2];
            a.v = v->data; a.v_nb1 = (int64_t)v->nb[1]; a.v_nb2 = (int64_t)v->nb[2];
            a.mask = m->data; a.mask_nb1 = (int64_t)m->nb[1];
            memcpy(&a.scale, &fa->op_params[0], 4);
            a.dst = (float *)fa->data;
            a.n_chunks = bc->cpu_threads;
            a.mode = 1;
            if (a.n_head % a.n_head_kv || a.n_head / a.n_head_kv > 4 || a.n_head_kv > DP_MAX_KV_HEADS || a.n_kv <= 0 || a.q_nb1 % 4 || a.q_nb2 % 4) return false;
            if (!flash_attn_fast_dims(&a, sms, 4, &P2.fd)) return false;
            P2.scale_log2 = a.scale * 1.4426950408889634f;
            if (*fa_splits && (*fa_splits != P2.fd.n_splits || *fa_heads != (int)a.n_head_kv)) return false;
            *fa_splits = P2.fd.n_splits;
            *fa_heads = (int)a.n_head_kv;
        }
        phases->push_back(P2);
        // phase 3: attn_output + residual
        DpPhase P3 = gemv_phase(DP_PRO_PLAIN, fa, nullptr, nullptr, (int)mmo->src[0]->ne[0]);
        P3.n_mat = 1;
        step_mat(&P3.mat[0], mmo, DP_EPI_ADD);
        P3.addend = (const float *)other_src(add1, mmo)->data;
        P3.sum = (float *)add1->data;
        close_phase(P3);
        // phase 4: norm | gate, up | silu(gate) * up
        DpPhase P4 = gemv_phase(DP_PRO_NORM, norm2->src[0], norm2, mul2, (int)E);
        P4.n_mat = 2;
        P4.pair = 1;
        step_mat(&P4.mat[0], mmg, DP_EPI_STORE);
        step_mat(&P4.mat[1], mmu, DP_EPI_STORE);
        P4.raw0 = (float *)mmg->data;
        P4.raw1 = (float *)mmu->data;
        P4.silu_out = (float *)silu->data;
        P4.h_out = (float *)gmul->data;
        P4.wide_end = bc->silu_wide ? (int)(mmg->ne[0] & ~(int64_t)15) : 0;
        close_phase(P4);
        // phase 5: ffn_down + residual
        DpPhase P5 = gemv_phase(DP_PRO_PLAIN, gmul, nullptr, nullptr, (int)mmd->src[0]->ne[0]);
        P5.n_mat = 1;
        step_mat(&P5.mat[0], mmd, DP_EPI_ADD);
        P5.addend = (const float *)add1->data;
        P5.sum = (float *)add2->data;
        close_phase(P5);
        if (n_layer == 0) *first = ops[c];
        n_layer++;
        c += 20;
    }
    if (n_layer == 0 || c + 4 > ops.size()) return false;
    // output norm, the wanted row, the output mat-mul
    const ggml_tensor *normf = T(c), *mulf = T(c + 1), *rows = T(c + 2), *mmout = T(c + 3);
    if (normf->op != GGML_OP_RMS_NORM || mulf->op != GGML_OP_MUL || rows->op != GGML_OP_GET_ROWS || mmout->op != GGML_OP_MUL_MAT) return false;
    if (!norm_pair_ok(normf, mulf) || rows->src[0] != mulf || rows->ne[1] != 1 || mmout->src[1] != rows) return false;
    {
        // the row GET_ROWS would copy is row 0 of a one-row tensor: the mat-mul reads the weighted norm where it is
        // (the copy, a node nothing else reads, is not made)
        const ggml_tensor *w = mmout->src[0];
        if (!supports_mul_mat(mmout, nullptr) || (w->type != B200_TYPE_Q4_K && w->type != B200_TYPE_Q6_K) || !is_tiled_tensor(w) || w->ne[2] != 1 ||
            w->ne[1] % TILE_ROWS || mmout->ne[1] != 1 || ((uintptr_t)mmout->data & 15) || ((uintptr_t)rows->data & 15) || w->ne[0] != normf->ne[0])
            return false;
        DpPhase PF = gemv_phase(DP_PRO_NORM, normf->src[0], normf, mulf, (int)normf->ne[0]);
        PF.n_mat = 1;
        step_mat(&PF.mat[0], mmout, DP_EPI_STORE);
        close_phase(PF);
    }
    for (const DpPhase &P : *phases) {
        if (P.kind != DP_GEMV) continue;
        if (decode_persistent_work_bytes(P.k) > decode_persistent_work_limit()) return false;
        if (P.prologue == DP_PRO_NORM && P.k > decode_persistent_norm_max_k()) return false;
    }
    *last = ops[c + 3] + 1;
    return true;
}

// the plan of the list being computed (built on first sight, rebuilt when an address it holds has been re-allocated)
static int step_plan_for(BackendCtx *bc, const ggml_cgraph *g, uint64_t key, BackendCtx::StepPlan **out) {
    *out = nullptr;
    if (!bc->persistent_decode || numerics_mode() != 1 || bc->tp != nullptr || key == 0) return B200_STATUS_SUCCESS;
    BackendCtx::StepPlan *p = nullptr;
    for (auto &cand : bc->plans)
        if (cand.key == key) p = &cand;
    static uint64_t clock = 0;
    if (p && p->generation == bc->generation) {
        p->used = ++clock;
        if (p->usable) *out = p;
        return B200_STATUS_SUCCESS;
    }
    if (!p) {
        if (bc->plans.size() >= 16) {
            auto lru = std::min_element(bc->plans.begin(), bc->plans.end(),
                                        [](const BackendCtx::StepPlan &a, const BackendCtx::StepPlan &b) { return a.used < b.used; });
            B200_CUDA(cudaStreamSynchronize(bc->stream));
            if (lru->dev_phases) cudaFree(lru->dev_phases);
            if (lru->dev_sync) cudaFree(lru->dev_sync);
            if (lru->dev_partial) cudaFree(lru->dev_partial);
            bc->plans.erase(lru);
        }
        bc->plans.emplace_back();
        p = &bc->plans.back();
        p->key = key;
    }
    p->used = ++clock;
    p->generation = bc->generation;
    p->usable = false;
    std::vector<DpPhase> phases;
    int fa_splits = 0, fa_heads = 0;
    if (!match_decode_step(bc, g, &phases, &p->first, &p->last, &fa_splits, &fa_heads)) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaStreamSynchronize(bc->stream));   // a launch in flight may still read the previous phase list
    if (p->dev_phases) cudaFree(p->dev_phases);
    if (p->dev_partial) cudaFree(p->dev_partial);
    p->dev_phases = nullptr;
    p->dev_partial = nullptr;
    if (!p->dev_sync) B200_CUDA(cudaMalloc((void **)&p->dev_sync, sizeof(DpSync)));
    B200_CUDA(cudaMalloc((void **)&p->dev_partial, decode_persistent_attn_partial_bytes(fa_heads, fa_splits, 128)));
    for (DpPhase &P : phases)
        if (P.kind == DP_ATTN) {
            P.partial = p->dev_partial;
            P.counters = p->dev_sync->fa_counters;
        }
    B200_CUDA(cudaMalloc((void **)&p->dev_phases, phases.size() * sizeof(DpPhase)));
    B200_CUDA(cudaMemcpy(p->dev_phases, phases.data(), phases.size() * sizeof(DpPhase), cudaMemcpyHostToDevice));
    p->n_phases = (int)phases.size();
    p->usable = true;
    *out = p;
    return B200_STATUS_SUCCESS;
}

// Issues the launches of every node, in order, on the backend's stream.
static int run_nodes(BackendCtx *bc, ggml_cgraph *g) {
    bc->act_src = nullptr;   // tensors may have been rewritten between graphs
    struct FaScope {         // one mask serves every layer of this node list: attention may reuse what it derives from it
        FaScope() { flash_attn_graph_scope(true); }
        ~FaScope() { flash_attn_graph_scope(false); }
    } fa_scope;
    const void *fa_mask = nullptr;   // the mask the attention nodes so far have read
    size_t fa_mask_bytes = 0;
    std::vector<int> silu_of(g->n_nodes, -1);   // silu_of[j] = i: MUL node j also computes SILU node i
    std::vector<char> done(g->n_nodes, 0);      // mat-mul nodes that ran early, with a sibling
    PendingPrologue pending;                    // a norm / silu that rides with the mat-mul that follows it
    BackendCtx::StepPlan *plan = nullptr;
    {
        int rc = step_plan_for(bc, g, bc->current_key, &plan);
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    for (int i = 0; i < g->n_nodes; i++) {
        const ggml_tensor *op = g->nodes[i];
        B200_REQUIRE(op != nullptr, "graph_compute: node %d is null", i);
        if (done[i]) continue;
        if (plan && i == plan->first) {   // the layers and the output mat-mul of a one-token step: one kernel
            bc->act_src = nullptr;
            int rc = launch_decode_persistent(plan->dev_phases, plan->n_phases, plan->dev_sync, bc->stream);
            if (rc != B200_STATUS_SUCCESS) return rc;
            i = plan->last - 1;
            continue;
        }
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
        const bool is_alias = op->op == GGML_OP_NONE || op->op == GGML_OP_RESHAPE || op->op == GGML_OP_VIEW ||
                              op->op == GGML_OP_PERMUTE || op->op == GGML_OP_TRANSPOSE;
        if (is_alias) continue;
        const ggml_tensor *next = i + 1 < g->n_nodes ? g->nodes[i + 1] : nullptr;
        // a node that writes over the rows whose quantized copy is cached ends that copy's life
        if (bc->act_src && op->data && ranges_overlap(op->data, ggml_nbytes(op), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
            bc->act_src = nullptr;
        if (op->type == B200_TYPE_I32 && in_our_buffer(op)) shadow_drop(bctx(op->buffer), op->data);
        if (op->op == GGML_OP_FLASH_ATTN_EXT) {
            if (op->src[3] && op->src[3]->data) {
                fa_mask = op->src[3]->data;
                fa_mask_bytes = ggml_nbytes(op->src[3]);
            }
        } else if (fa_mask && op->data && ranges_overlap(op->data, ggml_nbytes(op), fa_mask, fa_mask_bytes)) {
            flash_attn_graph_scope(true);   // a node rewrites the mask: what attention derived from it is stale
            fa_mask = nullptr;
        }
        int rc = B200_STATUS_SUCCESS;
        if (debug_skip(op)) continue;
        switch (op->op) {
            case GGML_OP_MUL_MAT:
                if (pending.active || (bc->fuse_prologue && (prologue_mask() & 1) && multi_candidate(op) && ((uintptr_t)op->src[1]->data & 15) == 0 &&
                                       !(bc->act_src == op->src[1]->data && bc->act_m == 1 && bc->act_k == op->src[1]->ne[0] &&
                                         bc->act_kind == B200_ACT_Q8_K))) {
                    // the op in front of this mat-mul (or just the quantization of its activations) runs in its kernel
                    b200_act_prologue pro;
                    const ggml_tensor *act_tensor = op->src[1];
                    if (pending.active) {
                        pro = pending.pro;
                        act_tensor = pending.act_tensor;
                        pending.active = false;
                    } else {
                        memset(&pro, 0, sizeof(pro));
                        pro.mode = B200_ACT_PRO_PLAIN;
                        pro.x = (const float *)op->src[1]->data;
                    }
                    if (next && fuses_mul_mat_add(op, next)) {
                        if (bc->act_src && ranges_overlap(next->data, ggml_nbytes(next), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                            bc->act_src = nullptr;
                        rc = compute_mul_mat_row_fused(bc, g, i, nullptr, 0, next, pro, act_tensor);
                        i++;
                    } else {
                        int sib[2];
                        const int n_sib = bc->fuse_siblings ? find_sibling_mat_muls(g, i, sib) : 0;
                        rc = compute_mul_mat_row_fused(bc, g, i, sib, n_sib, nullptr, pro, act_tensor);
                        for (int e = 0; e < n_sib; e++) done[sib[e]] = 1;
                    }
                } else if (next && fuses_mul_mat_add(op, next) && supports_mul_mat(op, nullptr)) {
                    if (bc->act_src && ranges_overlap(next->data, ggml_nbytes(next), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                        bc->act_src = nullptr;
                    rc = compute_mul_mat_add(bc, op, next);
                    i++;
                } else if (next && bc->fuse_siblings && fuses_mul_mat_rows_add(op, next)) {
                    rc = compute_mul_mat_rows_add(bc, op, next);
                    if (bc->act_src && ranges_overlap(next->data, ggml_nbytes(next), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                        bc->act_src = nullptr;
                    i++;
                } else {
                    int sib[2];
                    const bool rows = op->src[1]->ne[1] > 1;
                    const int n_sib = bc->fuse_siblings ? find_sibling_mat_muls(g, i, sib, rows) : 0;
                    if (n_sib > 0) {
                        rc = rows ? compute_mul_mat_multi_rows(bc, g, i, sib, n_sib) : compute_mul_mat_multi(bc, g, i, sib, n_sib);
                        for (int e = 0; e < n_sib; e++) done[sib[e]] = 1;
                    } else {
                        rc = compute_mul_mat(bc, op);
                    }
                }
                break;
            case GGML_OP_MUL_MAT_ID: rc = compute_mul_mat_id(bc, op); break;
            case GGML_OP_FLASH_ATTN_EXT: rc = compute_flash(bc, op); break;
            case GGML_OP_RMS_NORM:
                if (next && fuses_norm_mul(op, next)) {
                    if (bc->act_src && ranges_overlap(next->data, ggml_nbytes(next), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                        bc->act_src = nullptr;
                    const ggml_tensor *x = op->src[0];
                    const bool al = (((uintptr_t)x->data | (uintptr_t)op->data | (uintptr_t)next->data | (uintptr_t)next->src[1]->data) & 15) == 0;
                    const int jm = bc->fuse_prologue && al && (prologue_mask() & 10) ? fusable_row_mat_mul(g, i + 1, next) : -1;
                    // every CTA of the mat-mul redoes the norm: worth it while the launch is a wave or two of CTAs
                    if (jm >= 0 && ((prologue_mask() & 8) || row_tiles_of(g, jm) <= 2 * 148)) {
                        memset(&pending.pro, 0, sizeof(pending.pro));
                        pending.pro.mode = B200_ACT_PRO_NORM;
                        pending.pro.x = (const float *)x->data;
                        pending.pro.w = (const float *)next->src[1]->data;
                        pending.pro.eps = param_f32(op, 0);
                        pending.pro.y = (float *)op->data;
                        pending.pro.y_mul = (float *)next->data;
                        pending.act_tensor = next;
                        pending.active = true;
                    } else {
                        rc = compute_rms_norm(bc, op, next, upcoming_q8_K_kind(g, i + 1, next));
                    }
                    i++;
                } else {
                    rc = compute_rms_norm(bc, op, nullptr, upcoming_q8_K_kind(g, i, op));
                }
                break;
            case GGML_OP_UNARY: {
                const int j = find_silu_mul(g, i);
                if (j > 0) silu_of[j] = i;   // runs with node j
                else rc = compute_silu(bc, op, nullptr, upcoming_q8_K_kind(g, i, op));
                break;
            }
            case GGML_OP_MUL:
                if (silu_of[i] >= 0) {
                    const ggml_tensor *silu = g->nodes[silu_of[i]];
                    if (bc->act_src && ranges_overlap(silu->data, ggml_nbytes(silu), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                        bc->act_src = nullptr;
                    const bool al = (((uintptr_t)silu->src[0]->data | (uintptr_t)silu->data | (uintptr_t)op->data | (uintptr_t)op->src[1]->data) & 15) == 0;
                    if (bc->fuse_prologue && (prologue_mask() & 4) && al && fusable_row_mat_mul(g, i, op) >= 0) {
                        memset(&pending.pro, 0, sizeof(pending.pro));
                        pending.pro.mode = B200_ACT_PRO_SILU;
                        pending.pro.x = (const float *)silu->src[0]->data;
                        pending.pro.w = (const float *)op->src[1]->data;
                        pending.pro.wide = bc->silu_wide;
                        pending.pro.y = (float *)silu->data;
                        pending.pro.y_mul = (float *)op->data;
                        pending.act_tensor = op;
                        pending.active = true;
                    } else {
                        rc = compute_silu(bc, silu, op, upcoming_q8_K_kind(g, i, op));
                    }
                } else {
                    rc = compute_binary(bc, op);
                }
                break;
            case GGML_OP_ADD: rc = compute_binary(bc, op); break;
            case GGML_OP_ROPE:
            case GGML_OP_SET_ROWS: {
                GlueBatch gb;
                int members[2 * GLUE_BATCH_MAX];
                const int nm = bc->fuse_glue ? gather_glue_batch(bc, g, i, done, &gb, members) : 0;
                if (nm >= 2) {
                    for (int e = 0; e < nm; e++) {
                        const ggml_tensor *mem = g->nodes[members[e]];
                        if (bc->act_src && ranges_overlap(mem->data, ggml_nbytes(mem), bc->act_src, (size_t)bc->act_ld * bc->act_m * 4))
                            bc->act_src = nullptr;
                        if (members[e] != i) done[members[e]] = 1;
                    }
                    rc = launch_glue_batch(gb, bc->stream);
                } else {
                    rc = op->op == GGML_OP_ROPE ? compute_rope(bc, op) : compute_set_rows(bc, op);
                }
                break;
            }
            case GGML_OP_GET_ROWS: rc = compute_get_rows(bc, op); break;
            case GGML_OP_ARGMAX: rc = compute_argmax(bc, op); break;
            case B200_OP_TP_ALL_REDUCE:
                rc = tp_all_reduce(bc->tp, (float *)op->data, (int64_t)(ggml_nbytes(op) / 4), bc->stream, &bc->capturable);
                break;
            case B200_OP_TP_ALL_GATHER:
                rc = tp_all_gather_rows(bc->tp, (const float *)op->src[0]->data, (float *)op->data, op->src[0]->ne[0], op->src[0]->ne[1],
                                        op->src[1] ? (float *)op->src[1]->data : nullptr, bc->stream, &bc->capturable);
                break;
            default: break;
        }
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    return B200_STATUS_SUCCESS;
}

// ---- CUDA graphs over repeated node lists ---------------------------------------------------------------
// A decode loop hands the same node list (same tensors, same addresses) to graph_compute once per token,
// and at one token the list is launch-bound: some hundreds of kernels of a few microseconds each.  The
// second time a list comes by unchanged its launches are captured into a CUDA graph (the programmatic
// dependent-launch edges between the kernels included), and from then on one graph launch replays them.
// What a launch reads from the host while being issued must therefore not depend on values that change
// between tokens: positions reach ROPE through the position tensor on the device (rope_prepare), and the
// key below covers everything else a node's launches are derived from.
// the key is recomputed on every graph_compute, over a few hundred KB for a 32-layer decode step: eight bytes
// per multiply (a byte-wise chain of dependent multiplies cost a third of a millisecond per token)
static uint64_t fnv(uint64_t h, const void *p, size_t n) {
    const uint8_t *b = (const uint8_t *)p;
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
        uint64_t w;
        memcpy(&w, b + i, 8);
        h = (h ^ w) * 0x9e3779b97f4a7c15ull;
        h ^= h >> 32;
    }
    for (; i < n; i++) h = (h ^ b[i]) * 0x100000001b3ull;
    return h;
}
static uint64_t node_list_key(const BackendCtx *bc, const ggml_cgraph *g) {
    uint64_t h = 0xcbf29ce484222325ull;
    h = fnv(h, &bc->cpu_threads, sizeof(int));
    h = fnv(h, &bc->silu_wide, sizeof(int));
    h = fnv(h, &bc->fuse_siblings, sizeof(bool));
    h = fnv(h, &bc->fuse_glue, sizeof(bool));
    h = fnv(h, &bc->fuse_prologue, sizeof(bool));
    const int numerics = numerics_mode();
    h = fnv(h, &numerics, sizeof(int));
    h = fnv(h, &bc->persistent_decode, sizeof(bool));
    h = fnv(h, &g->n_nodes, sizeof(int));
    for (int i = 0; i < g->n_nodes; i++) {
        const ggml_tensor *t = g->nodes[i];
        if (!t) continue;
        h = fnv(h, &t->type, sizeof(int32_t));
        h = fnv(h, t->ne, sizeof(t->ne) + sizeof(t->nb));
        h = fnv(h, &t->op, sizeof(int32_t) + sizeof(t->op_params));
        h = fnv(h, &t->data, sizeof(void *));
        for (int s = 0; s < GGML_MAX_SRC; s++) {
            const ggml_tensor *src = t->src[s];
            if (!src) continue;
            h = fnv(h, &src->type, sizeof(int32_t));
            h = fnv(h, src->ne, sizeof(src->ne) + sizeof(src->nb));
            h = fnv(h, &src->data, sizeof(void *));
        }
    }
    return h;
}
static void drop_captured(BackendCtx *bc) {
    for (auto &c : bc->captured)
        if (c.exec) cudaGraphExecDestroy(c.exec);
    bc->captured.clear();
}

static int backend_graph_compute(ggml_backend_t be, ggml_cgraph *g) {
    BackendCtx *bc = (BackendCtx *)be->context;
    B200_REQUIRE(g != nullptr && (g->n_nodes == 0 || g->nodes != nullptr), "graph_compute: null graph");
    B200_CUDA(cudaSetDevice(bc->device));
    bc->capturable = true;
    for (int i = 0; i < g->n_nodes; i++) {
        const ggml_tensor *op = g->nodes[i];
        if (op && op->op == GGML_OP_ROPE && supports_glue(op, nullptr)) {
            int rc = rope_prepare(bc, op);
            if (rc != B200_STATUS_SUCCESS) return rc;
        }
        if (op && (op->op == B200_OP_TP_ALL_REDUCE || op->op == B200_OP_TP_ALL_GATHER)) {
            B200_REQUIRE(bc->tp != nullptr, "graph_compute: node %d is a tensor-parallel collective, but no group is attached to this backend", i);
            if (bc->tp->hook) bc->capturable = false;   // the exchange happens on the host
        }
    }
    bc->current_key = 0;
    if (g->n_nodes < 6) return run_nodes(bc, g);
    const uint64_t key = node_list_key(bc, g);
    bc->current_key = key;
    {
        // a step the persistent kernel takes is a handful of launches: nothing to capture
        BackendCtx::StepPlan *plan = nullptr;
        int rc = step_plan_for(bc, g, key, &plan);
        if (rc != B200_STATUS_SUCCESS) return rc;
        if (plan) return run_nodes(bc, g);
    }
    if (!bc->graphs_enabled || !bc->capturable) return run_nodes(bc, g);

    const unsigned long long sgen = scratch_generation();
    BackendCtx::CapturedGraph *c = nullptr;
    for (auto &cand : bc->captured)
        if (cand.key == key) c = &cand;
    static uint64_t clock = 0;
    if (!c) {   // first sight: run it eagerly (this also grows every scratch block to its working size)
        if (bc->captured.size() >= GRAPHS_KEPT) {
            auto lru = std::min_element(bc->captured.begin(), bc->captured.end(),
                                        [](const BackendCtx::CapturedGraph &a, const BackendCtx::CapturedGraph &b) { return a.used < b.used; });
            if (lru->exec) cudaGraphExecDestroy(lru->exec);
            bc->captured.erase(lru);
        }
        bc->captured.emplace_back();
        bc->captured.back().key = key;
        bc->captured.back().used = ++clock;
        return run_nodes(bc, g);
    }
    c->used = ++clock;
    if (c->refused) return run_nodes(bc, g);
    if (c->exec && (c->generation != bc->generation || c->scratch_generation != sgen)) {
        cudaGraphExecDestroy(c->exec);   // an address it holds has been re-allocated since
        c->exec = nullptr;
    }
    if (!c->exec) {
        cudaGraph_t graph = nullptr;
        B200_CUDA(cudaStreamBeginCapture(bc->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = run_nodes(bc, g);
        const cudaError_t e = cudaStreamEndCapture(bc->stream, &graph);
        if (rc != B200_STATUS_SUCCESS || e != cudaSuccess || !graph || !bc->capturable || scratch_generation() != sgen) {
            if (graph) cudaGraphDestroy(graph);
            cudaGetLastError();
            c->refused = true;
            if (rc != B200_STATUS_SUCCESS && e == cudaSuccess) return rc;   // the list itself is at fault
            return run_nodes(bc, g);
        }
        const cudaError_t ei = cudaGraphInstantiate(&c->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ei != cudaSuccess) {
            cudaGetLastError();
            c->exec = nullptr;
            c->refused = true;
            return run_nodes(bc, g);
        }
        c->generation = bc->generation;
        c->scratch_generation = sgen;
    }
    B200_CUDA(cudaGraphLaunch(c->exec, bc->stream));
    return B200_STATUS_SUCCESS;
}

// ---- backend -------------------------------------------------------------------------------------
static const char *backend_get_name(ggml_backend_t be) { return ((BackendCtx *)be->context)->name.c_str(); }
static void backend_free(ggml_backend_t be) {
    BackendCtx *bc = (BackendCtx *)be->context;
    cudaSetDevice(bc->device);
    cudaStreamSynchronize(bc->stream);
    drop_captured(bc);
    for (auto &pl : bc->plans) {
        if (pl.dev_phases) cudaFree(pl.dev_phases);
        if (pl.dev_sync) cudaFree(pl.dev_sync);
        if (pl.dev_partial) cudaFree(pl.dev_partial);
    }
    if (bc->act) cudaFree(bc->act);
    if (bc->rope_dev) cudaFree(bc->rope_dev);
    for (auto &t : bc->rope_by_pos)
        if (t.dev) cudaFree(t.dev);
    cudaStreamDestroy(bc->stream);
    delete bc;
    delete be;
}
// Ordered on the backend's stream, before the next graph_compute; the host memory may be reused on return (the
// runtime stages a pageable source before it returns).  Quantized tensors take the synchronous path: they are
// re-ordered by a kernel on the way in.
static void backend_set_tensor_async(ggml_backend_t be, ggml_tensor *t, const void *data, size_t offset, size_t size) {
    if (!t->buffer || size == 0) return;
    if (is_tiled_tensor(t) || !in_our_buffer(t)) {
        t->buffer->iface.set_tensor(t->buffer, t, data, offset, size);
        return;
    }
    BackendCtx *bc = (BackendCtx *)be->context;
    BufferCtx *c = bctx(t->buffer);
    cudaSetDevice(bc->device);
    shadow_note_write(c, t, data, offset, size);
    if (b200_memcpy_h2d((uint8_t *)t->data + offset, data, size, bc->stream) != B200_STATUS_SUCCESS) note(c, "set_tensor_async");
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
static void *backend_get_stream(ggml_backend_t be) { return be ? (void *)((BackendCtx *)be->context)->stream : nullptr; }
static void backend_set_tp(ggml_backend_t be, void *group) {
    if (!be) return;
    BackendCtx *bc = (BackendCtx *)be->context;
    bc->tp = (TpGroup *)group;
    bc->generation++;   // captured graphs hold the old group's buffers
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
    BackendCtx *bc = new BackendCtx();
    bc->device = dev;
    bc->cpu_threads = 8;
    bc->name = std::string("B200") + std::to_string(dev);
    bc->silu_wide = b200_host_silu_is_wide();
    {
        const char *e = getenv("B200_CUDA_GRAPHS");
        if (e && e[0] == '0') bc->graphs_enabled = false;
        const char *fs = getenv("B200_FUSE_SIBLINGS");
        if (fs && fs[0] == '0') bc->fuse_siblings = false;
        const char *fg = getenv("B200_FUSE_GLUE");
        if (fg && fg[0] == '0') bc->fuse_glue = false;
        const char *fp = getenv("B200_FUSE_PROLOGUE");
        if (fp && fp[0] == '0') bc->fuse_prologue = false;
        const char *dp = getenv("B200_DECODE_PERSISTENT");
        if (dp) bc->persistent_decode = dp[0] == '1';
    }
    if (cudaStreamCreateWithFlags(&bc->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        set_error("init_backend: cannot create a stream on device %d", dev);
        delete bc;
        return nullptr;
    }
    if (params) {   // "cpu_threads=<n>"
        const char *p = strstr(params, "cpu_threads=");
        if (p) {
            int n = atoi(p + 12);
            if (n > 0) bc->cpu_threads = n;
        }
        p = strstr(params, "silu_wide=");
        if (p) bc->silu_wide = atoi(p + 10) != 0;
        p = strstr(params, "cuda_graphs=");
        if (p) bc->graphs_enabled = atoi(p + 12) != 0;
        p = strstr(params, "fuse_siblings=");
        if (p) bc->fuse_siblings = atoi(p + 14) != 0;
        p = strstr(params, "fuse_glue=");
        if (p) bc->fuse_glue = atoi(p + 10) != 0;
        p = strstr(params, "fuse_prologue=");
        if (p) bc->fuse_prologue = atoi(p + 14) != 0;
        p = strstr(params, "decode_persistent=");
        if (p) bc->persistent_decode = atoi(p + 18) != 0;
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
    if (name && strcmp(name, "b200_backend_get_stream") == 0) return (void *)backend_get_stream;
    if (name && strcmp(name, "b200_backend_set_tp") == 0) return (void *)backend_set_tp;
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
