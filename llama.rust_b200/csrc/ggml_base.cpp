// The libggml-base-shaped export set (include/ggml_base_b200.h): metadata contexts, the graph builder,
// buffer / device / registry pass-throughs over the plug-in vtables, a host "CPU" device that owns memory
// but computes nothing, and a one-device scheduler that runs every node on the B200 backend.
//
// Mirrors the call surface the reference resolves by name (crates/ggml/src/sysffi.rs:458-629) and the order
// its ForeignExecutor drives it in (crates/ggml/src/backend_emit.rs:439-572, 895-1042).  Host code only.
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <strings.h>
#include <algorithm>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "ggml_base_b200.h"

namespace {

void log_line(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    fprintf(stderr, "ggml-b200: ");
    vfprintf(stderr, fmt, ap);
    fprintf(stderr, "\n");
    va_end(ap);
}

// ---- types: (block elements, block bytes) by enum ggml_type value ----------------------------------------
struct TypeTraits {
    int blck;
    int size;
};
TypeTraits type_traits(int type) {
    switch (type) {
        case 0: return {1, 4};      // F32
        case 1: return {1, 2};      // F16
        case 2: return {32, 18};    // Q4_0
        case 3: return {32, 20};    // Q4_1
        case 6: return {32, 22};    // Q5_0
        case 7: return {32, 24};    // Q5_1
        case 8: return {32, 34};    // Q8_0
        case 9: return {32, 36};    // Q8_1
        case 10: return {256, 84};  // Q2_K
        case 11: return {256, 110}; // Q3_K
        case 12: return {256, 144}; // Q4_K
        case 13: return {256, 176}; // Q5_K
        case 14: return {256, 210}; // Q6_K
        case 15: return {256, 292}; // Q8_K
        case 24: return {1, 1};     // I8
        case 25: return {1, 2};     // I16
        case 26: return {1, 4};     // I32
        case 27: return {1, 8};     // I64
        case 28: return {1, 8};     // F64
        case 30: return {1, 2};     // BF16
        case 39: return {32, 17};   // MXFP4
        default: return {0, 0};
    }
}

size_t tensor_nbytes(const ggml_tensor *t) {
    const TypeTraits tt = type_traits(t->type);
    if (tt.blck == 0) return 0;
    for (int i = 0; i < GGML_MAX_DIMS; i++)
        if (t->ne[i] <= 0) return 0;
    // ggml_nbytes: the span from the first to the last byte, strides honoured
    size_t n = tt.blck == 1 ? (size_t)t->ne[0] * t->nb[0] : (size_t)t->ne[0] * t->nb[0] / tt.blck;
    for (int i = 1; i < GGML_MAX_DIMS; i++) n += (size_t)(t->ne[i] - 1) * t->nb[i];
    return n;
}

bool is_view_op(int op) { return op == GGML_OP_RESHAPE || op == GGML_OP_VIEW || op == GGML_OP_PERMUTE || op == GGML_OP_TRANSPOSE; }

constexpr size_t OBJECT_SIZE = 32, MEM_ALIGN = 16;
size_t pad_to(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

// ---- contexts ---------------------------------------------------------------------------------------------
struct ggml_context {
    uint8_t *mem = nullptr;
    size_t size = 0, used = 0;
    bool owned = false, no_alloc = true;
    std::vector<std::unordered_set<const ggml_tensor *> *> visited_sets;   // one per graph built here
    void *take(size_t bytes) {
        const size_t need = pad_to(bytes, MEM_ALIGN) + OBJECT_SIZE;
        if (used + need > size) return nullptr;
        void *p = mem + used + OBJECT_SIZE;
        used += need;
        return p;
    }
};

// the graph: the public leading fields, then the visited set
struct GraphImpl {
    ggml_cgraph g;
    std::unordered_set<const ggml_tensor *> *visited;
};

extern "C" {

struct ggml_context *ggml_init(struct ggml_init_params params) {
    ggml_context *ctx = new ggml_context;
    ctx->size = pad_to(params.mem_size, MEM_ALIGN);
    ctx->no_alloc = params.no_alloc;
    if (params.mem_buffer) {
        ctx->mem = (uint8_t *)params.mem_buffer;
    } else {
        ctx->mem = (uint8_t *)aligned_alloc(64, pad_to(ctx->size ? ctx->size : 64, 64));
        ctx->owned = true;
    }
    if (!ctx->mem) {
        delete ctx;
        return nullptr;
    }
    return ctx;
}

void ggml_free(struct ggml_context *ctx) {
    if (!ctx) return;
    for (auto *v : ctx->visited_sets) delete v;
    if (ctx->owned) free(ctx->mem);
    delete ctx;
}

size_t ggml_tensor_overhead(void) { return OBJECT_SIZE + sizeof(ggml_tensor); }

size_t ggml_graph_overhead_custom(size_t size, bool grads) {
    size_t n = sizeof(GraphImpl) + 2 * size * sizeof(ggml_tensor *);
    if (grads) n += 2 * size * sizeof(ggml_tensor *);
    return OBJECT_SIZE + pad_to(n, MEM_ALIGN);
}

struct ggml_tensor *ggml_new_tensor(struct ggml_context *ctx, int type, int n_dims, const int64_t *ne) {
    const TypeTraits tt = type_traits(type);
    if (!ctx || tt.blck == 0 || n_dims < 1 || n_dims > GGML_MAX_DIMS || ne[0] % tt.blck != 0) {
        log_line("ggml_new_tensor: bad arguments (type %d, %d dims)", type, n_dims);
        return nullptr;
    }
    int64_t e[GGML_MAX_DIMS] = {1, 1, 1, 1};
    for (int i = 0; i < n_dims; i++) e[i] = ne[i];
    size_t data = 0;
    if (!ctx->no_alloc) {
        data = (size_t)(e[0] / tt.blck) * tt.size;
        for (int i = 1; i < GGML_MAX_DIMS; i++) data *= (size_t)e[i];
    }
    ggml_tensor *t = (ggml_tensor *)ctx->take(sizeof(ggml_tensor) + data);
    if (!t) {
        log_line("ggml_new_tensor: context of %zu bytes is full", ctx->size);
        return nullptr;
    }
    memset(t, 0, sizeof(ggml_tensor));
    t->type = type;
    for (int i = 0; i < GGML_MAX_DIMS; i++) t->ne[i] = e[i];
    t->nb[0] = (size_t)tt.size;
    t->nb[1] = t->nb[0] * (size_t)(e[0] / tt.blck);
    for (int i = 2; i < GGML_MAX_DIMS; i++) t->nb[i] = t->nb[i - 1] * (size_t)e[i - 1];
    if (data) t->data = (uint8_t *)t + sizeof(ggml_tensor);
    return t;
}

struct ggml_tensor *ggml_set_name(struct ggml_tensor *tensor, const char *name) {
    if (tensor && name) {
        strncpy(tensor->name, name, GGML_MAX_NAME - 1);
        tensor->name[GGML_MAX_NAME - 1] = 0;
    }
    return tensor;
}
void ggml_set_input(struct ggml_tensor *tensor) {
    if (tensor) tensor->flags |= GGML_TENSOR_FLAG_INPUT;
}
void ggml_set_output(struct ggml_tensor *tensor) {
    if (tensor) tensor->flags |= GGML_TENSOR_FLAG_OUTPUT;
}

struct ggml_cgraph *ggml_new_graph_custom(struct ggml_context *ctx, size_t size, bool grads) {
    if (!ctx) return nullptr;
    size_t bytes = sizeof(GraphImpl) + 2 * size * sizeof(ggml_tensor *);
    if (grads) bytes += 2 * size * sizeof(ggml_tensor *);
    GraphImpl *gi = (GraphImpl *)ctx->take(bytes);
    if (!gi) {
        log_line("ggml_new_graph_custom: context of %zu bytes is full", ctx->size);
        return nullptr;
    }
    memset(gi, 0, bytes);
    ggml_tensor **slots = (ggml_tensor **)(gi + 1);
    gi->g.size = (int)size;
    gi->g.nodes = slots;
    gi->g.leafs = slots + size;
    if (grads) {
        gi->g.grads = slots + 2 * size;
        gi->g.grad_accs = slots + 3 * size;
    }
    ctx->visited_sets.push_back(new std::unordered_set<const ggml_tensor *>());   // freed with the context
    gi->visited = ctx->visited_sets.back();
    return &gi->g;
}

static void visit(GraphImpl *gi, ggml_tensor *t) {
    if (!t || gi->visited->count(t)) return;
    gi->visited->insert(t);
    for (int i = 0; i < GGML_MAX_SRC; i++) visit(gi, t->src[i]);
    ggml_cgraph &g = gi->g;
    if (t->op == GGML_OP_NONE && !(t->flags & GGML_TENSOR_FLAG_PARAM)) {
        if (g.n_leafs >= g.size) {
            log_line("ggml_build_forward_expand: more than %d leafs", g.size);
            return;
        }
        if (!t->name[0]) snprintf(t->name, GGML_MAX_NAME, "leaf_%d", g.n_leafs);
        g.leafs[g.n_leafs++] = t;
    } else {
        if (g.n_nodes >= g.size) {
            log_line("ggml_build_forward_expand: more than %d nodes", g.size);
            return;
        }
        if (!t->name[0]) snprintf(t->name, GGML_MAX_NAME, "node_%d", g.n_nodes);
        g.nodes[g.n_nodes++] = t;
    }
}

void ggml_build_forward_expand(struct ggml_cgraph *cgraph, struct ggml_tensor *tensor) {
    if (cgraph && tensor) visit((GraphImpl *)cgraph, tensor);
}
int ggml_graph_n_nodes(struct ggml_cgraph *cgraph) { return cgraph ? cgraph->n_nodes : 0; }
struct ggml_tensor *ggml_graph_node(struct ggml_cgraph *cgraph, int i) {
    if (!cgraph) return nullptr;
    if (i < 0) i += cgraph->n_nodes;
    return i >= 0 && i < cgraph->n_nodes ? cgraph->nodes[i] : nullptr;
}
struct ggml_tensor **ggml_graph_nodes(struct ggml_cgraph *cgraph) { return cgraph ? cgraph->nodes : nullptr; }

int64_t ggml_time_us(void) {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// ---- buffers ------------------------------------------------------------------------------------------------
ggml_backend_buffer_t ggml_backend_buft_alloc_buffer(ggml_backend_buffer_type_t buft, size_t size) {
    return buft && buft->iface.alloc_buffer ? buft->iface.alloc_buffer(buft, size) : nullptr;
}
size_t ggml_backend_buft_get_alignment(ggml_backend_buffer_type_t buft) {
    return buft && buft->iface.get_alignment ? buft->iface.get_alignment(buft) : 32;
}
size_t ggml_backend_buft_get_max_size(ggml_backend_buffer_type_t buft) {
    return buft && buft->iface.get_max_size ? buft->iface.get_max_size(buft) : SIZE_MAX;
}
size_t ggml_backend_buft_get_alloc_size(ggml_backend_buffer_type_t buft, const struct ggml_tensor *tensor) {
    if (buft && buft->iface.get_alloc_size) return buft->iface.get_alloc_size(buft, tensor);
    return tensor_nbytes(tensor);
}
void ggml_backend_buffer_free(ggml_backend_buffer_t buffer) {
    if (buffer && buffer->iface.free_buffer) buffer->iface.free_buffer(buffer);
}
void *ggml_backend_buffer_get_base(ggml_backend_buffer_t buffer) {
    return buffer && buffer->iface.get_base ? buffer->iface.get_base(buffer) : nullptr;
}
void ggml_backend_buffer_clear(ggml_backend_buffer_t buffer, uint8_t value) {
    if (buffer && buffer->iface.clear) buffer->iface.clear(buffer, value);
}
void ggml_backend_buffer_set_usage(ggml_backend_buffer_t buffer, int usage) {
    if (buffer) buffer->usage = usage;
}

static ggml_backend_buffer_t buffer_of(const ggml_tensor *t) { return t->view_src ? t->view_src->buffer : t->buffer; }

void ggml_backend_tensor_set(struct ggml_tensor *tensor, const void *data, size_t offset, size_t size) {
    ggml_backend_buffer_t buf = tensor ? buffer_of(tensor) : nullptr;
    if (!buf || !tensor->data) {
        log_line("ggml_backend_tensor_set: tensor '%s' has no storage", tensor ? tensor->name : "(null)");
        return;
    }
    if (size) buf->iface.set_tensor(buf, tensor, data, offset, size);
}
void ggml_backend_tensor_get(const struct ggml_tensor *tensor, void *data, size_t offset, size_t size) {
    ggml_backend_buffer_t buf = tensor ? buffer_of(tensor) : nullptr;
    if (!buf || !tensor->data) {
        log_line("ggml_backend_tensor_get: tensor '%s' has no storage", tensor ? tensor->name : "(null)");
        return;
    }
    if (size) buf->iface.get_tensor(buf, tensor, data, offset, size);
}
int ggml_backend_tensor_alloc(ggml_backend_buffer_t buffer, struct ggml_tensor *tensor, void *addr) {
    if (!buffer || !tensor || !addr) return GGML_STATUS_ALLOC_FAILED;
    tensor->buffer = buffer;
    tensor->data = addr;
    return buffer->iface.init_tensor ? buffer->iface.init_tensor(buffer, tensor) : GGML_STATUS_SUCCESS;
}
int ggml_backend_view_init(struct ggml_tensor *tensor) {
    if (!tensor || !tensor->view_src || !tensor->view_src->buffer || !tensor->view_src->data) return GGML_STATUS_ALLOC_FAILED;
    tensor->buffer = tensor->view_src->buffer;
    tensor->data = (uint8_t *)tensor->view_src->data + tensor->view_offs;
    return tensor->buffer->iface.init_tensor ? tensor->buffer->iface.init_tensor(tensor->buffer, tensor) : GGML_STATUS_SUCCESS;
}

}  // extern "C"

// ---- the host device: memory only --------------------------------------------------------------------------
namespace {

struct HostBuffer {
    void *base;
    bool owned;
};

ggml_backend_buffer_type g_host_buft;
ggml_backend_device g_host_dev;
ggml_backend_reg g_host_reg;
int g_host_threads = 8;   // what "ggml_backend_set_n_threads" on the CPU backend last asked for

void host_free(ggml_backend_buffer_t b) {
    HostBuffer *h = (HostBuffer *)b->context;
    if (h->owned) free(h->base);
    delete h;
    delete b;
}
void *host_base(ggml_backend_buffer_t b) { return ((HostBuffer *)b->context)->base; }
void host_memset(ggml_backend_buffer_t, ggml_tensor *t, uint8_t v, size_t off, size_t n) { memset((uint8_t *)t->data + off, v, n); }
void host_set(ggml_backend_buffer_t, ggml_tensor *t, const void *d, size_t off, size_t n) { memcpy((uint8_t *)t->data + off, d, n); }
void host_get(ggml_backend_buffer_t, const ggml_tensor *t, void *d, size_t off, size_t n) { memcpy(d, (const uint8_t *)t->data + off, n); }
void host_clear(ggml_backend_buffer_t b, uint8_t v) { memset(host_base(b), v, b->size); }

ggml_backend_buffer_t host_make(void *base, size_t size, bool owned) {
    ggml_backend_buffer_t b = new ggml_backend_buffer;
    memset(b, 0, sizeof(*b));
    b->iface.free_buffer = host_free;
    b->iface.get_base = host_base;
    b->iface.memset_tensor = host_memset;
    b->iface.set_tensor = host_set;
    b->iface.get_tensor = host_get;
    b->iface.clear = host_clear;
    b->buft = &g_host_buft;
    b->context = new HostBuffer{base, owned};
    b->size = size;
    return b;
}
const char *host_buft_name(ggml_backend_buffer_type_t) { return "CPU"; }
ggml_backend_buffer_t host_buft_alloc(ggml_backend_buffer_type_t, size_t size) {
    void *p = aligned_alloc(64, pad_to(size ? size : 64, 64));
    return p ? host_make(p, size, true) : nullptr;
}
size_t host_buft_align(ggml_backend_buffer_type_t) { return 32; }
bool host_buft_is_host(ggml_backend_buffer_type_t) { return true; }

// the host backend exists so that a scheduler can be handed [gpu, cpu]; it runs nothing
const char *host_backend_name(ggml_backend_t) { return "CPU"; }
void host_backend_free(ggml_backend_t b) { delete b; }
void host_backend_sync(ggml_backend_t) {}
int host_backend_compute(ggml_backend_t, ggml_cgraph *g) {
    if (g && g->n_nodes > 0) {
        log_line("the CPU device of this library holds memory only: it cannot compute '%s'", g->nodes[0]->name);
        return GGML_STATUS_BACKEND_ERROR;
    }
    return GGML_STATUS_SUCCESS;
}
const char *host_dev_name(ggml_backend_dev_t) { return "CPU"; }
const char *host_dev_desc(ggml_backend_dev_t) { return "host memory (no compute)"; }
void host_dev_memory(ggml_backend_dev_t, size_t *fr, size_t *total) { *fr = *total = 0; }
int host_dev_type(ggml_backend_dev_t) { return GGML_BACKEND_DEVICE_TYPE_CPU; }
void host_dev_props(ggml_backend_dev_t d, ggml_backend_dev_props *p) {
    memset(p, 0, sizeof(*p));
    p->name = host_dev_name(d);
    p->description = host_dev_desc(d);
    p->type = GGML_BACKEND_DEVICE_TYPE_CPU;
    p->caps.buffer_from_host_ptr = true;
}
ggml_backend_t host_dev_init(ggml_backend_dev_t d, const char *) {
    ggml_backend_t b = new ggml_backend;
    memset(b, 0, sizeof(*b));
    b->iface.get_name = host_backend_name;
    b->iface.free = host_backend_free;
    b->iface.synchronize = host_backend_sync;
    b->iface.graph_compute = host_backend_compute;
    b->device = d;
    return b;
}
ggml_backend_buffer_type_t host_dev_buft(ggml_backend_dev_t) { return &g_host_buft; }
ggml_backend_buffer_t host_dev_from_ptr(ggml_backend_dev_t, void *p, size_t size, size_t) { return host_make(p, size, false); }
bool host_dev_supports_op(ggml_backend_dev_t, const ggml_tensor *op) { return op && (op->op == GGML_OP_NONE || is_view_op(op->op)); }
bool host_dev_supports_buft(ggml_backend_dev_t, ggml_backend_buffer_type_t t) { return t == &g_host_buft; }
bool host_dev_offload(ggml_backend_dev_t, const ggml_tensor *) { return false; }

const char *host_reg_name(ggml_backend_reg_t) { return "CPU"; }
size_t host_reg_count(ggml_backend_reg_t) { return 1; }
ggml_backend_dev_t host_reg_dev(ggml_backend_reg_t, size_t i) { return i == 0 ? &g_host_dev : nullptr; }
// ggml_backend_set_n_threads on the CPU backend: the thread count the CPU side would run with, which is the
// count whose split-KV attention arithmetic the device reproduces; the scheduler hands it to its backend
void host_set_n_threads(ggml_backend_t, int n) {
    if (n > 0) g_host_threads = n;
}
void *host_reg_proc(ggml_backend_reg_t, const char *name) {
    if (name && strcmp(name, "ggml_backend_set_n_threads") == 0) return (void *)host_set_n_threads;
    return nullptr;
}

struct Registry {
    std::vector<ggml_backend_dev_t> devs;
    Registry() {
        g_host_buft.iface.get_name = host_buft_name;
        g_host_buft.iface.alloc_buffer = host_buft_alloc;
        g_host_buft.iface.get_alignment = host_buft_align;
        g_host_buft.iface.is_host = host_buft_is_host;
        g_host_buft.device = &g_host_dev;
        g_host_dev.iface.get_name = host_dev_name;
        g_host_dev.iface.get_description = host_dev_desc;
        g_host_dev.iface.get_memory = host_dev_memory;
        g_host_dev.iface.get_type = host_dev_type;
        g_host_dev.iface.get_props = host_dev_props;
        g_host_dev.iface.init_backend = host_dev_init;
        g_host_dev.iface.get_buffer_type = host_dev_buft;
        g_host_dev.iface.buffer_from_host_ptr = host_dev_from_ptr;
        g_host_dev.iface.supports_op = host_dev_supports_op;
        g_host_dev.iface.supports_buft = host_dev_supports_buft;
        g_host_dev.iface.offload_op = host_dev_offload;
        g_host_dev.reg = &g_host_reg;
        g_host_reg.api_version = GGML_BACKEND_API_VERSION;
        g_host_reg.iface.get_name = host_reg_name;
        g_host_reg.iface.get_device_count = host_reg_count;
        g_host_reg.iface.get_device = host_reg_dev;
        g_host_reg.iface.get_proc_address = host_reg_proc;
        // GPU devices first: the order ggml registers its backends in
        ggml_backend_reg_t cuda = ggml_backend_init();
        if (cuda && cuda->iface.get_device_count)
            for (size_t i = 0; i < cuda->iface.get_device_count(cuda); i++) devs.push_back(cuda->iface.get_device(cuda, i));
        devs.push_back(&g_host_dev);
    }
};
Registry &registry() {
    static Registry r;
    return r;
}

}  // namespace

extern "C" {

ggml_backend_buffer_t ggml_backend_cpu_buffer_from_ptr(void *ptr, size_t size) {
    registry();
    return ptr ? host_make(ptr, size, false) : nullptr;
}
ggml_backend_buffer_type_t ggml_backend_cpu_buffer_type(void) {
    registry();
    return &g_host_buft;
}

size_t ggml_backend_dev_count(void) { return registry().devs.size(); }
ggml_backend_dev_t ggml_backend_dev_get(size_t index) { return index < registry().devs.size() ? registry().devs[index] : nullptr; }
const char *ggml_backend_dev_name(ggml_backend_dev_t device) { return device && device->iface.get_name ? device->iface.get_name(device) : ""; }
ggml_backend_dev_t ggml_backend_dev_by_name(const char *name) {
    if (!name) return nullptr;
    for (ggml_backend_dev_t d : registry().devs)
        if (strcasecmp(ggml_backend_dev_name(d), name) == 0) return d;
    // a registry's own name ("B200") stands for its first device ("B2000")
    for (ggml_backend_dev_t d : registry().devs)
        if (d->reg && d->reg->iface.get_name && strcasecmp(d->reg->iface.get_name(d->reg), name) == 0) return d;
    return nullptr;
}
ggml_backend_dev_t ggml_backend_dev_by_type(int type) {
    for (ggml_backend_dev_t d : registry().devs)
        if (d->iface.get_type && d->iface.get_type(d) == type) return d;
    return nullptr;
}
void ggml_backend_free(ggml_backend_t backend) {
    if (backend && backend->iface.free) backend->iface.free(backend);
}
ggml_backend_t ggml_backend_dev_init(ggml_backend_dev_t device, const char *params) {
    return device && device->iface.init_backend ? device->iface.init_backend(device, params) : nullptr;
}
ggml_backend_buffer_type_t ggml_backend_dev_buffer_type(ggml_backend_dev_t device) {
    return device && device->iface.get_buffer_type ? device->iface.get_buffer_type(device) : nullptr;
}
ggml_backend_reg_t ggml_backend_dev_backend_reg(ggml_backend_dev_t device) { return device ? device->reg : nullptr; }
void *ggml_backend_reg_get_proc_address(ggml_backend_reg_t reg, const char *name) {
    return reg && reg->iface.get_proc_address ? reg->iface.get_proc_address(reg, name) : nullptr;
}
void ggml_backend_load_all_from_path(const char *) { registry(); }

void ggml_backend_synchronize(ggml_backend_t backend) {
    if (backend && backend->iface.synchronize) backend->iface.synchronize(backend);
}
void ggml_backend_tensor_set_async(ggml_backend_t backend, struct ggml_tensor *tensor, const void *data, size_t offset, size_t size) {
    if (backend && backend->iface.set_tensor_async) backend->iface.set_tensor_async(backend, tensor, data, offset, size);
    else ggml_backend_tensor_set(tensor, data, offset, size);
}
void ggml_backend_tensor_get_async(ggml_backend_t backend, const struct ggml_tensor *tensor, void *data, size_t offset, size_t size) {
    if (backend && backend->iface.get_tensor_async) backend->iface.get_tensor_async(backend, tensor, data, offset, size);
    else ggml_backend_tensor_get(tensor, data, offset, size);
}

size_t b200_gpu_layer_start(size_t n_layer_all, int32_t n_gpu_layers) {
    if (n_gpu_layers <= 0) return SIZE_MAX;
    const int64_t start = (int64_t)n_layer_all + 1 - (int64_t)n_gpu_layers;
    return (size_t)(start > 0 ? start : 0);
}
bool b200_layer_on_gpu(size_t n_layer_all, int32_t n_gpu_layers, size_t il) {
    return il >= b200_gpu_layer_start(n_layer_all, n_gpu_layers) && il < n_layer_all + 1;
}

}  // extern "C"

// ---- the scheduler ----------------------------------------------------------------------------------------
struct ggml_backend_sched {
    std::vector<ggml_backend_t> backends;
    ggml_backend_t gpu = nullptr;
    ggml_backend_dev_t gpu_dev = nullptr;
    ggml_backend_buffer_type_t gpu_buft = nullptr;
    ggml_backend_buffer_t compute = nullptr;          // step tensors
    std::vector<ggml_backend_buffer_t> weight_bufs;    // device mirrors of host weights, kept
    ggml_backend_buffer_t stage = nullptr;             // device mirrors of other host sources, per step
    struct Mirror {
        ggml_tensor t;       // the device twin's metadata (owned here)
        const ggml_tensor *host;
        bool weights;
    };
    std::unordered_map<const void *, Mirror *> mirrors;   // by host data pointer
    struct Patch {
        ggml_tensor *node;
        int slot;
        ggml_tensor *host, *twin;
    };
    std::vector<Patch> patches;
    std::vector<Mirror *> step_uploads;
    std::unordered_map<const ggml_tensor *, ggml_backend_t> pinned;
    ggml_backend_sched_copy_callback copy_cb = nullptr;
    void *copy_user = nullptr;
    int threads_applied = 0;
};

namespace {

bool is_host_buffer(ggml_backend_buffer_t b) { return b && b->buft && b->buft->iface.is_host && b->buft->iface.is_host(b->buft); }

void apply_threads(ggml_backend_sched *s) {
    if (s->threads_applied == g_host_threads || !s->gpu_dev || !s->gpu_dev->reg) return;
    typedef void (*set_fn)(ggml_backend_t, int);
    set_fn f = (set_fn)ggml_backend_reg_get_proc_address(s->gpu_dev->reg, "b200_backend_set_cpu_threads");
    if (f) f(s->gpu, g_host_threads);
    s->threads_applied = g_host_threads;
}

}  // namespace

extern "C" {

ggml_backend_sched_t ggml_backend_sched_new(ggml_backend_t *backends, ggml_backend_buffer_type_t *bufts, int n_backends, size_t, bool,
                                            bool) {
    if (!backends || n_backends < 1) return nullptr;
    ggml_backend_sched *s = new ggml_backend_sched;
    for (int i = 0; i < n_backends; i++) {
        ggml_backend_t b = backends[i];
        s->backends.push_back(b);
        if (!s->gpu && b && b->device && b->device->iface.get_type && b->device->iface.get_type(b->device) == GGML_BACKEND_DEVICE_TYPE_GPU) {
            s->gpu = b;
            s->gpu_dev = b->device;
            s->gpu_buft = bufts && bufts[i] ? bufts[i] : ggml_backend_dev_buffer_type(b->device);
        }
    }
    if (!s->gpu || !s->gpu_buft) {
        log_line("ggml_backend_sched_new: no GPU backend among the %d given; this scheduler runs every node on the device", n_backends);
        delete s;
        return nullptr;
    }
    return s;
}

// per-step mirrors go; weight mirrors stay
static void drop_step_mirrors(ggml_backend_sched *s) {
    s->patches.clear();
    s->step_uploads.clear();
    for (auto it = s->mirrors.begin(); it != s->mirrors.end();) {
        if (!it->second->weights) {
            delete it->second;
            it = s->mirrors.erase(it);
        } else {
            ++it;
        }
    }
}

void ggml_backend_sched_reset(ggml_backend_sched_t s) {
    if (!s) return;
    drop_step_mirrors(s);
    s->pinned.clear();
}

void ggml_backend_sched_free(ggml_backend_sched_t s) {
    if (!s) return;
    for (auto &kv : s->mirrors) delete kv.second;
    s->mirrors.clear();
    ggml_backend_buffer_free(s->compute);
    ggml_backend_buffer_free(s->stage);
    for (ggml_backend_buffer_t b : s->weight_bufs) ggml_backend_buffer_free(b);
    delete s;
}

bool ggml_backend_sched_alloc_graph(ggml_backend_sched_t s, struct ggml_cgraph *g) {
    if (!s || !g) return false;
    drop_step_mirrors(s);
    const size_t align = ggml_backend_buft_get_alignment(s->gpu_buft);
    // every node has to run on the device
    for (int i = 0; i < g->n_nodes; i++) {
        ggml_tensor *t = g->nodes[i];
        if (!s->gpu_dev->iface.supports_op(s->gpu_dev, t)) {
            log_line("sched_alloc_graph: node %d '%s' (op %d) is not supported by %s and there is no CPU compute path", i, t->name, t->op,
                     ggml_backend_dev_name(s->gpu_dev));
            return false;
        }
        ggml_backend_buffer_t dstbuf = t->view_src ? t->view_src->buffer : t->buffer;
        if (is_host_buffer(dstbuf)) {
            log_line("sched_alloc_graph: node %d '%s' writes into a host buffer; results have to live on the device", i, t->name);
            return false;
        }
    }
    // step tensors without storage: one bump allocation in the compute buffer
    std::vector<ggml_tensor *> need;
    size_t total = 0;
    auto plan = [&](ggml_tensor *t) {
        if (t->data || t->view_src) return;
        total = pad_to(total, align) + ggml_backend_buft_get_alloc_size(s->gpu_buft, t);
        need.push_back(t);
    };
    for (int i = 0; i < g->n_leafs; i++) plan(g->leafs[i]);
    for (int i = 0; i < g->n_nodes; i++) plan(g->nodes[i]);
    total = pad_to(total, align) + align;
    if (!s->compute || s->compute->size < total) {
        ggml_backend_buffer_free(s->compute);
        s->compute = ggml_backend_buft_alloc_buffer(s->gpu_buft, total);
        if (!s->compute) {
            log_line("sched_alloc_graph: could not allocate a compute buffer of %zu bytes", total);
            return false;
        }
        ggml_backend_buffer_set_usage(s->compute, GGML_BACKEND_BUFFER_USAGE_COMPUTE);
    }
    uint8_t *base = (uint8_t *)ggml_backend_buffer_get_base(s->compute);
    size_t off = 0;
    for (ggml_tensor *t : need) {
        off = pad_to(off, align);
        if (ggml_backend_tensor_alloc(s->compute, t, base + off) != GGML_STATUS_SUCCESS) return false;
        off += ggml_backend_buft_get_alloc_size(s->gpu_buft, t);
    }
    // views, in graph order so that a view of a view finds its parent placed
    auto place_view = [&](ggml_tensor *t) -> bool {
        if (t->data || !t->view_src) return true;
        return ggml_backend_view_init(t) == GGML_STATUS_SUCCESS;
    };
    for (int i = 0; i < g->n_leafs; i++)
        if (!place_view(g->leafs[i])) return false;
    for (int i = 0; i < g->n_nodes; i++)
        if (!place_view(g->nodes[i])) {
            log_line("sched_alloc_graph: view '%s' has no placed parent", g->nodes[i]->name);
            return false;
        }
    // sources in host buffers get a device twin
    size_t stage_total = 0;
    std::vector<ggml_backend_sched::Mirror *> fresh_stage;
    for (int i = 0; i < g->n_nodes; i++) {
        ggml_tensor *t = g->nodes[i];
        for (int k = 0; k < GGML_MAX_SRC; k++) {
            ggml_tensor *src = t->src[k];
            if (!src || !is_host_buffer(buffer_of(src))) continue;
            if (src->view_src && src->nb[0] != (size_t)type_traits(src->type).size) {
                log_line("sched_alloc_graph: source '%s' of '%s' is a strided view of host memory", src->name, t->name);
                return false;
            }
            ggml_backend_sched::Mirror *m = nullptr;
            auto it = s->mirrors.find(src->data);
            if (it != s->mirrors.end()) {
                m = it->second;
            } else {
                m = new ggml_backend_sched::Mirror;
                m->t = *src;
                m->host = src;
                m->t.buffer = nullptr;
                m->t.data = nullptr;
                m->t.view_src = nullptr;
                m->t.view_offs = 0;
                m->t.op = GGML_OP_NONE;
                for (int j = 0; j < GGML_MAX_SRC; j++) m->t.src[j] = nullptr;
                m->weights = buffer_of(src)->usage == GGML_BACKEND_BUFFER_USAGE_WEIGHTS;
                const size_t bytes = ggml_backend_buft_get_alloc_size(s->gpu_buft, &m->t);
                if (m->weights) {
                    ggml_backend_buffer_t wb = ggml_backend_buft_alloc_buffer(s->gpu_buft, bytes + align);
                    if (!wb || ggml_backend_tensor_alloc(wb, &m->t, ggml_backend_buffer_get_base(wb)) != GGML_STATUS_SUCCESS) {
                        log_line("sched_alloc_graph: no device memory for the mirror of '%s' (%zu bytes)", src->name, bytes);
                        delete m;
                        return false;
                    }
                    ggml_backend_buffer_set_usage(wb, GGML_BACKEND_BUFFER_USAGE_WEIGHTS);
                    s->weight_bufs.push_back(wb);
                    // the whole weight goes up now, unless a copy callback takes care of the part that is used
                    if (!(s->copy_cb && s->copy_cb(s->gpu, src, &m->t, g, s->copy_user)))
                        ggml_backend_tensor_set(&m->t, src->data, 0, tensor_nbytes(src));
                } else {
                    stage_total = pad_to(stage_total, align) + bytes;
                    fresh_stage.push_back(m);
                }
                s->mirrors[src->data] = m;
            }
            s->patches.push_back({t, k, src, &m->t});
            if (!m->weights && std::find(s->step_uploads.begin(), s->step_uploads.end(), m) == s->step_uploads.end())
                s->step_uploads.push_back(m);
        }
    }
    if (!fresh_stage.empty()) {
        stage_total = pad_to(stage_total, align) + align;
        if (!s->stage || s->stage->size < stage_total) {
            ggml_backend_buffer_free(s->stage);
            s->stage = ggml_backend_buft_alloc_buffer(s->gpu_buft, stage_total);
            if (!s->stage) return false;
        }
        uint8_t *sb = (uint8_t *)ggml_backend_buffer_get_base(s->stage);
        size_t so = 0;
        for (ggml_backend_sched::Mirror *m : fresh_stage) {
            so = pad_to(so, align);
            if (ggml_backend_tensor_alloc(s->stage, &m->t, sb + so) != GGML_STATUS_SUCCESS) return false;
            so += ggml_backend_buft_get_alloc_size(s->gpu_buft, &m->t);
        }
    }
    return true;
}

int ggml_backend_sched_graph_compute(ggml_backend_sched_t s, struct ggml_cgraph *g) {
    if (!s || !g) return GGML_STATUS_BACKEND_ERROR;
    apply_threads(s);
    // host sources that are not weights are read at compute time (the host may have rewritten them)
    for (auto *m : s->step_uploads) ggml_backend_tensor_set(&m->t, m->host->data, 0, tensor_nbytes(m->host));
    for (const auto &p : s->patches) p.node->src[p.slot] = p.twin;
    const int st = s->gpu->iface.graph_compute(s->gpu, g);
    for (const auto &p : s->patches) p.node->src[p.slot] = p.host;
    return st;
}

void ggml_backend_sched_synchronize(ggml_backend_sched_t s) {
    if (s) ggml_backend_synchronize(s->gpu);
}
void ggml_backend_sched_set_tensor_backend(ggml_backend_sched_t s, struct ggml_tensor *node, ggml_backend_t backend) {
    if (s && node) s->pinned[node] = backend;   // recorded and reported back; every node still runs on the device
}
ggml_backend_t ggml_backend_sched_get_tensor_backend(ggml_backend_sched_t s, struct ggml_tensor *node) {
    if (!s || !node) return nullptr;
    if (node->op == GGML_OP_NONE) {
        // a leaf lives where its buffer is
        ggml_backend_buffer_t b = buffer_of(node);
        if (is_host_buffer(b))
            for (ggml_backend_t be : s->backends)
                if (be != s->gpu) return be;
    }
    return s->gpu;
}
int ggml_backend_sched_get_n_backends(ggml_backend_sched_t s) { return s ? (int)s->backends.size() : 0; }
ggml_backend_t ggml_backend_sched_get_backend(ggml_backend_sched_t s, int i) {
    return s && i >= 0 && i < (int)s->backends.size() ? s->backends[i] : nullptr;
}
size_t ggml_backend_sched_get_buffer_size(ggml_backend_sched_t s, ggml_backend_t backend) {
    return s && backend == s->gpu && s->compute ? s->compute->size : 0;
}
void ggml_backend_sched_set_copy_callback(ggml_backend_sched_t s, ggml_backend_sched_copy_callback callback, void *user_data) {
    if (!s) return;
    s->copy_cb = callback;
    s->copy_user = user_data;
}

}  // extern "C"
