// GGUF v3 files: a reader over a memory map, a writer, and the loader that feeds a llama-architecture file
// to the decode driver.
//
// Layout as the reference reads and writes it (crates/ggml/src/gguf.rs:388-655, gguf_write.rs:35-193): magic
// "GGUF", u32 version, u64 tensor count, u64 key count; keys (u64-length string, u32 value type, value; arrays
// carry their element type and a u64 count); tensor infos (name, u32 n_dims, u64 dims, u32 ggml type, u64
// offset into the data section); zero padding to the alignment (general.alignment, default 32); tensor data,
// each tensor padded to the alignment.  Little-endian throughout.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"
#include "llama_b200.h"

using namespace b200;

namespace {

enum : uint32_t { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };

size_t scalar_size(uint32_t t) {
    switch (t) {
        case T_U8: case T_I8: case T_BOOL: return 1;
        case T_U16: case T_I16: return 2;
        case T_U32: case T_I32: case T_F32: return 4;
        case T_U64: case T_I64: case T_F64: return 8;
        default: return 0;
    }
}

// bytes of ne[0] elements of a ggml type (crates/ggml/src/types.rs:172 row_size); 0 = a type this library does not know
size_t gguf_row_size(int type, int64_t ne0) {
    switch (type) {
        case B200_TYPE_F32: case B200_TYPE_I32: return (size_t)ne0 * 4;
        case B200_TYPE_F16: return (size_t)ne0 * 2;
        case B200_TYPE_I64: return (size_t)ne0 * 8;
        case B200_TYPE_Q4_0: return ne0 % 32 ? 0 : (size_t)ne0 / 32 * 18;
        case B200_TYPE_Q8_0: return ne0 % 32 ? 0 : (size_t)ne0 / 32 * 34;
        case B200_TYPE_MXFP4: return ne0 % 32 ? 0 : (size_t)ne0 / 32 * 17;
        case B200_TYPE_Q4_K: return ne0 % 256 ? 0 : (size_t)ne0 / 256 * 144;
        case B200_TYPE_Q6_K: return ne0 % 256 ? 0 : (size_t)ne0 / 256 * 210;
        case B200_TYPE_Q8_K: return ne0 % 256 ? 0 : (size_t)ne0 / 256 * 292;
        default: return 0;
    }
}

struct Value {
    uint32_t type = 0, elem_type = 0;
    uint64_t count = 0;          // arrays
    const uint8_t *data = nullptr;   // scalars: the value; strings: the bytes; arrays: the first element
    uint64_t len = 0;            // strings: byte length; arrays: bytes of all elements
};

struct TensorInfo {
    std::string name;
    int type = 0;
    int n_dims = 0;
    int64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;
    size_t nbytes = 0;
};

}  // namespace

struct b200_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32, data_offset = 0;
    std::vector<std::pair<std::string, Value>> kv;
    std::vector<TensorInfo> tensors;
    const Value *find(const char *key) const {
        for (auto &p : kv)
            if (p.first == key) return &p.second;
        return nullptr;
    }
};

namespace {

struct Cursor {
    const uint8_t *p, *end;
    bool ok = true;
    template <typename T> T get() {
        T v{};
        if ((size_t)(end - p) < sizeof(T)) { ok = false; return v; }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    bool skip(uint64_t n) {
        if ((uint64_t)(end - p) < n) { ok = false; return false; }
        p += n;
        return true;
    }
    bool str(std::string *s) {
        const uint64_t n = get<uint64_t>();
        if (!ok || (uint64_t)(end - p) < n) { ok = false; return false; }
        s->assign((const char *)p, n);
        p += n;
        return true;
    }
};

bool read_value(Cursor &c, uint32_t type, Value *v, int depth) {
    v->type = type;
    if (type == T_STR) {
        v->len = c.get<uint64_t>();
        v->data = c.p;
        return c.skip(v->len);
    }
    if (type == T_ARR) {
        if (depth > 0) { c.ok = false; return false; }   // the format has no arrays of arrays
        v->elem_type = c.get<uint32_t>();
        v->count = c.get<uint64_t>();
        v->data = c.p;
        if (v->elem_type == T_STR) {
            for (uint64_t i = 0; i < v->count && c.ok; i++) c.skip(c.get<uint64_t>());
        } else {
            const size_t es = scalar_size(v->elem_type);
            if (!es || v->count > (uint64_t)(c.end - c.p) / es) { c.ok = false; return false; }
            c.skip(v->count * es);
        }
        v->len = (uint64_t)(c.p - v->data);
        return c.ok;
    }
    const size_t es = scalar_size(type);
    if (!es) { c.ok = false; return false; }
    v->data = c.p;
    return c.skip(es);
}

template <typename T> T scalar(const Value *v) {
    T x{};
    memcpy(&x, v->data, sizeof(T));
    return x;
}

}  // namespace

extern "C" {

int b200_gguf_open(const char *path, b200_gguf **out) {
    B200_REQUIRE(path != nullptr && out != nullptr, "gguf_open: null argument");
    *out = nullptr;
    std::unique_ptr<b200_gguf> g(new b200_gguf());
    g->fd = open(path, O_RDONLY);
    B200_REQUIRE(g->fd >= 0, "gguf_open: cannot open %s", path);
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) {
        close(g->fd);
        B200_REQUIRE(false, "gguf_open: %s is too short to be a GGUF file", path);
    }
    g->size = (size_t)st.st_size;
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        close(g->fd);
        B200_REQUIRE(false, "gguf_open: cannot map %s", path);
    }
    g->map = (const uint8_t *)m;
    auto fail = [&](const char *why) {
        set_error("gguf_open: %s: %s", path, why);
        munmap((void *)g->map, g->size);
        close(g->fd);
        return B200_STATUS_BACKEND_ERROR;
    };
    Cursor c{g->map, g->map + g->size};
    if (memcmp(c.p, "GGUF", 4) != 0) return fail("bad magic");
    c.skip(4);
    g->version = c.get<uint32_t>();
    if (g->version != 2 && g->version != 3) return fail("unsupported version (2 and 3 are read)");
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (n_tensors > g->size || n_kv > g->size) return fail("implausible counts");
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key;
        Value v;
        if (!c.str(&key)) return fail("truncated key");
        // the reference refuses empty and repeated keys (crates/ggml/src/gguf.rs:509-512)
        if (key.empty()) return fail("empty key");
        for (auto &o : g->kv)
            if (o.first == key) return fail("duplicate key");
        const uint32_t type = c.get<uint32_t>();
        if (!read_value(c, type, &v, 0)) return fail("truncated or malformed value");
        g->kv.emplace_back(std::move(key), v);
    }
    if (const Value *a = g->find("general.alignment")) {
        if (a->type == T_U32) g->alignment = scalar<uint32_t>(a);
        if (g->alignment == 0 || (g->alignment & (g->alignment - 1))) return fail("general.alignment is not a power of two");
    }
    for (uint64_t i = 0; i < n_tensors; i++) {
        TensorInfo t;
        if (!c.str(&t.name)) return fail("truncated tensor name");
        t.n_dims = (int)c.get<uint32_t>();
        if (!c.ok || t.n_dims < 1 || t.n_dims > 4) return fail("tensor with a bad dimension count");
        for (int d = 0; d < t.n_dims; d++) {
            t.ne[d] = (int64_t)c.get<uint64_t>();
            if (t.ne[d] < 0) return fail("tensor with a negative dimension");   // crates/ggml/src/gguf.rs:554
        }
        t.type = (int)c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail("truncated tensor info");
        for (auto &o : g->tensors)
            if (o.name == t.name) return fail("duplicate tensor name");
        const size_t rs = gguf_row_size(t.type, t.ne[0]);
        // 0 for types this library does not know; a product that does not fit size_t cannot be a tensor of this file
        size_t nb = rs;
        for (int d = 1; d < 4; d++)
            if (__builtin_mul_overflow(nb, (size_t)t.ne[d], &nb)) return fail("tensor size overflows");
        t.nbytes = nb;
        g->tensors.push_back(std::move(t));
    }
    const uint64_t meta = (uint64_t)(c.p - g->map);
    g->data_offset = (meta + g->alignment - 1) / g->alignment * g->alignment;
    if (g->data_offset > g->size) return fail("metadata runs past the end of the file");
    const uint64_t data_size = g->size - g->data_offset;
    for (auto &t : g->tensors)   // subtractions only: no sum that a huge offset could wrap
        if (t.offset % g->alignment || t.offset > data_size || t.nbytes > data_size - t.offset) return fail("tensor data outside the file or misaligned");
    *out = g.release();
    return B200_STATUS_SUCCESS;
}

void b200_gguf_close(b200_gguf *g) {
    if (!g) return;
    if (g->map) munmap((void *)g->map, g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int64_t b200_gguf_n_tensors(const b200_gguf *g) { return g ? (int64_t)g->tensors.size() : 0; }
int64_t b200_gguf_n_kv(const b200_gguf *g) { return g ? (int64_t)g->kv.size() : 0; }
uint32_t b200_gguf_version(const b200_gguf *g) { return g ? g->version : 0; }
uint64_t b200_gguf_data_offset(const b200_gguf *g) { return g ? g->data_offset : 0; }

int b200_gguf_tensor(const b200_gguf *g, int64_t i, const char **name, int *type, int64_t ne[4], const void **data, size_t *nbytes) {
    B200_REQUIRE(g != nullptr && i >= 0 && i < (int64_t)g->tensors.size(), "gguf_tensor: index out of range");
    const TensorInfo &t = g->tensors[i];
    if (name) *name = t.name.c_str();
    if (type) *type = t.type;
    if (ne) memcpy(ne, t.ne, sizeof(t.ne));
    if (data) *data = g->map + g->data_offset + t.offset;
    if (nbytes) *nbytes = t.nbytes;
    return B200_STATUS_SUCCESS;
}

int b200_gguf_find_tensor(const b200_gguf *g, const char *name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) return (int)i;
    return -1;
}

/* scalar getters: 0 on success, BACKEND_ERROR when the key is missing or of another type */
int b200_gguf_get_u32(const b200_gguf *g, const char *key, uint32_t *out) {
    const Value *v = g ? g->find(key) : nullptr;
    B200_REQUIRE(v != nullptr, "gguf: key %s not found", key);
    if (v->type == T_U32 || v->type == T_I32) *out = scalar<uint32_t>(v);
    else if (v->type == T_U16) *out = scalar<uint16_t>(v);
    else if (v->type == T_U8 || v->type == T_BOOL) *out = scalar<uint8_t>(v);
    else if (v->type == T_U64 || v->type == T_I64) *out = (uint32_t)scalar<uint64_t>(v);
    else if (v->type == T_ARR && v->count > 0 && (v->elem_type == T_U32 || v->elem_type == T_I32)) *out = scalar<uint32_t>(v);   // per-layer arrays: the first entry
    else B200_REQUIRE(false, "gguf: key %s is not an integer", key);
    return B200_STATUS_SUCCESS;
}
int b200_gguf_get_f32(const b200_gguf *g, const char *key, float *out) {
    const Value *v = g ? g->find(key) : nullptr;
    B200_REQUIRE(v != nullptr, "gguf: key %s not found", key);
    if (v->type == T_F32) *out = scalar<float>(v);
    else if (v->type == T_F64) *out = (float)scalar<double>(v);
    else B200_REQUIRE(false, "gguf: key %s is not a float", key);
    return B200_STATUS_SUCCESS;
}
int b200_gguf_get_str(const b200_gguf *g, const char *key, char *out, size_t out_len) {
    const Value *v = g ? g->find(key) : nullptr;
    B200_REQUIRE(v != nullptr, "gguf: key %s not found", key);
    B200_REQUIRE(v->type == T_STR, "gguf: key %s is not a string", key);
    B200_REQUIRE(out != nullptr && out_len > v->len, "gguf: buffer too small for %s", key);
    memcpy(out, v->data, v->len);
    out[v->len] = 0;
    return B200_STATUS_SUCCESS;
}
int64_t b200_gguf_arr_len(const b200_gguf *g, const char *key) {
    const Value *v = g ? g->find(key) : nullptr;
    return v && v->type == T_ARR ? (int64_t)v->count : -1;
}

}  // extern "C"

// ---- writer ------------------------------------------------------------------------------------------------
struct b200_gguf_writer {
    uint64_t alignment = 32;
    struct Kv { std::string key; uint32_t type; std::vector<uint8_t> bytes; };
    std::vector<Kv> kv;
    struct T { std::string name; int type; int64_t ne[4]; uint64_t offset; size_t nbytes; const void *data; };
    std::vector<T> tensors;
    void set(const char *key, uint32_t type, const void *p, size_t n) {
        for (auto &k : kv)
            if (k.key == key) { k.type = type; k.bytes.assign((const uint8_t *)p, (const uint8_t *)p + n); return; }
        kv.push_back({key, type, std::vector<uint8_t>((const uint8_t *)p, (const uint8_t *)p + n)});
    }
};

namespace {
void put(std::vector<uint8_t> &b, const void *p, size_t n) { b.insert(b.end(), (const uint8_t *)p, (const uint8_t *)p + n); }
template <typename T> void put(std::vector<uint8_t> &b, T v) { put(b, &v, sizeof(v)); }
int n_dims_of(const int64_t ne[4]) {
    int n = 1;
    for (int i = 1; i < 4; i++)
        if (ne[i] > 1) n = i + 1;
    return n;
}
}  // namespace

extern "C" {

int b200_gguf_writer_new(uint64_t alignment, b200_gguf_writer **out) {
    B200_REQUIRE(out != nullptr && alignment > 0 && (alignment & (alignment - 1)) == 0, "gguf_writer_new: the alignment must be a power of two");
    *out = new b200_gguf_writer();
    (*out)->alignment = alignment;
    return B200_STATUS_SUCCESS;
}
void b200_gguf_writer_free(b200_gguf_writer *w) { delete w; }

int b200_gguf_set_u32(b200_gguf_writer *w, const char *key, uint32_t v) { B200_REQUIRE(w && key && *key, "gguf_set: bad argument"); w->set(key, T_U32, &v, 4); return B200_STATUS_SUCCESS; }
int b200_gguf_set_f32(b200_gguf_writer *w, const char *key, float v) { B200_REQUIRE(w && key && *key, "gguf_set: bad argument"); w->set(key, T_F32, &v, 4); return B200_STATUS_SUCCESS; }
int b200_gguf_set_str(b200_gguf_writer *w, const char *key, const char *v) {
    B200_REQUIRE(w && key && *key && v, "gguf_set: bad argument");
    std::vector<uint8_t> b;
    put<uint64_t>(b, strlen(v));
    put(b, v, strlen(v));
    w->set(key, T_STR, b.data(), b.size());
    return B200_STATUS_SUCCESS;
}
/* arrays of one scalar type (elem_type: the GGUF value type id, e.g. 5 = i32, 6 = f32) */
int b200_gguf_set_arr(b200_gguf_writer *w, const char *key, uint32_t elem_type, const void *data, uint64_t count) {
    B200_REQUIRE(w && key && *key && (data || count == 0), "gguf_set: bad argument");
    const size_t es = scalar_size(elem_type);
    B200_REQUIRE(es != 0, "gguf_set_arr: element type %u is not a scalar", elem_type);
    std::vector<uint8_t> b;
    put<uint32_t>(b, elem_type);
    put<uint64_t>(b, count);
    put(b, data, es * count);
    w->set(key, T_ARR, b.data(), b.size());
    return B200_STATUS_SUCCESS;
}
int b200_gguf_set_arr_str(b200_gguf_writer *w, const char *key, const char *const *strs, uint64_t count) {
    B200_REQUIRE(w && key && *key && (strs || count == 0), "gguf_set: bad argument");
    std::vector<uint8_t> b;
    put<uint32_t>(b, T_STR);
    put<uint64_t>(b, count);
    for (uint64_t i = 0; i < count; i++) {
        put<uint64_t>(b, strlen(strs[i]));
        put(b, strs[i], strlen(strs[i]));
    }
    w->set(key, T_ARR, b.data(), b.size());
    return B200_STATUS_SUCCESS;
}

/* data must stay valid until b200_gguf_write */
int b200_gguf_add_tensor(b200_gguf_writer *w, const char *name, int type, const int64_t ne[4], const void *data, size_t nbytes) {
    B200_REQUIRE(w && name && ne && data, "gguf_add_tensor: null argument");
    for (auto &t : w->tensors) B200_REQUIRE(t.name != name, "gguf_add_tensor: duplicate tensor name %s", name);
    const size_t rs = gguf_row_size(type, ne[0]);
    B200_REQUIRE(rs != 0, "gguf_add_tensor: %s: type %d / row length %lld", name, type, (long long)ne[0]);
    B200_REQUIRE(nbytes == rs * (size_t)ne[1] * (size_t)ne[2] * (size_t)ne[3], "gguf_add_tensor: %s: %zu bytes given", name, nbytes);
    uint64_t offset = 0;
    if (!w->tensors.empty()) {
        const auto &p = w->tensors.back();
        offset = p.offset + (p.nbytes + w->alignment - 1) / w->alignment * w->alignment;
    }
    b200_gguf_writer::T t{name, type, {ne[0], ne[1], ne[2], ne[3]}, offset, nbytes, data};
    w->tensors.push_back(t);
    return B200_STATUS_SUCCESS;
}

int b200_gguf_write(const b200_gguf_writer *w, const char *path) {
    B200_REQUIRE(w && path, "gguf_write: null argument");
    std::vector<uint8_t> b;
    put(b, "GGUF", 4);
    put<uint32_t>(b, 3);
    put<uint64_t>(b, w->tensors.size());
    put<uint64_t>(b, w->kv.size());
    for (auto &k : w->kv) {
        put<uint64_t>(b, k.key.size());
        put(b, k.key.data(), k.key.size());
        put<uint32_t>(b, k.type);
        put(b, k.bytes.data(), k.bytes.size());
    }
    for (auto &t : w->tensors) {
        put<uint64_t>(b, t.name.size());
        put(b, t.name.data(), t.name.size());
        const int nd = n_dims_of(t.ne);
        put<uint32_t>(b, (uint32_t)nd);
        for (int d = 0; d < nd; d++) put<uint64_t>(b, (uint64_t)t.ne[d]);
        put<uint32_t>(b, (uint32_t)t.type);
        put<uint64_t>(b, t.offset);
    }
    b.resize((b.size() + w->alignment - 1) / w->alignment * w->alignment, 0);
    FILE *f = fopen(path, "wb");
    B200_REQUIRE(f != nullptr, "gguf_write: cannot create %s", path);
    bool ok = fwrite(b.data(), 1, b.size(), f) == b.size();
    const std::vector<uint8_t> zeros(w->alignment, 0);
    for (auto &t : w->tensors) {
        ok = ok && fwrite(t.data, 1, t.nbytes, f) == t.nbytes;
        const size_t pad = (t.nbytes + w->alignment - 1) / w->alignment * w->alignment - t.nbytes;
        ok = ok && fwrite(zeros.data(), 1, pad, f) == pad;
    }
    ok = fclose(f) == 0 && ok;
    B200_REQUIRE(ok, "gguf_write: short write to %s", path);
    return B200_STATUS_SUCCESS;
}

// ---- loader ------------------------------------------------------------------------------------------------
// The llama.* keys of crates/llama/src/model.rs (LlamaHparams::from_gguf) that the decode driver needs.
int b200_llama_load_gguf_tp(const char *path, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, int32_t tp_rank,
                            int32_t tp_size, const void *id128, b200_llama **out) {
    B200_REQUIRE(out != nullptr, "llama_load_gguf: null argument");
    *out = nullptr;
    b200_gguf *g = nullptr;
    int rc = b200_gguf_open(path, &g);
    if (rc != B200_STATUS_SUCCESS) return rc;
    struct Closer { b200_gguf *g; ~Closer() { b200_gguf_close(g); } } closer{g};
    char arch[64] = "";
    rc = b200_gguf_get_str(g, "general.architecture", arch, sizeof(arch));
    if (rc != B200_STATUS_SUCCESS) return rc;
    B200_REQUIRE(strcmp(arch, "llama") == 0, "llama_load_gguf: architecture %s is not llama", arch);
    b200_llama_hparams hp;
    memset(&hp, 0, sizeof(hp));
    uint32_t u = 0;
    auto need = [&](const char *key, int32_t *dst) {
        int r = b200_gguf_get_u32(g, key, &u);
        if (r == B200_STATUS_SUCCESS) *dst = (int32_t)u;
        return r;
    };
    if ((rc = need("llama.block_count", &hp.n_layer)) || (rc = need("llama.embedding_length", &hp.n_embd)) ||
        (rc = need("llama.feed_forward_length", &hp.n_ff)) || (rc = need("llama.attention.head_count", &hp.n_head)))
        return rc;
    hp.n_head_kv = hp.n_head;
    if (g->find("llama.attention.head_count_kv")) need("llama.attention.head_count_kv", &hp.n_head_kv);
    B200_REQUIRE(hp.n_head > 0, "llama_load_gguf: llama.attention.head_count is zero");
    hp.n_embd_head = hp.n_embd / hp.n_head;
    if (g->find("llama.attention.key_length")) need("llama.attention.key_length", &hp.n_embd_head);
    hp.n_ctx_train = 4096;
    if (g->find("llama.context_length")) need("llama.context_length", &hp.n_ctx_train);
    if (g->find("llama.rope.scaling.original_context_length")) need("llama.rope.scaling.original_context_length", &hp.n_ctx_train);
    hp.norm_rms_eps = 1e-5f;
    if (g->find("llama.attention.layer_norm_rms_epsilon")) b200_gguf_get_f32(g, "llama.attention.layer_norm_rms_epsilon", &hp.norm_rms_eps);
    hp.rope_freq_base = 10000.0f;
    if (g->find("llama.rope.freq_base")) b200_gguf_get_f32(g, "llama.rope.freq_base", &hp.rope_freq_base);
    hp.rope_freq_scale = 1.0f;
    hp.rope_mode = 0;   // llama: adjacent pairs
    const int tok = b200_gguf_find_tensor(g, "token_embd.weight");
    B200_REQUIRE(tok >= 0, "llama_load_gguf: %s has no token_embd.weight", path);
    hp.n_vocab = (int32_t)g->tensors[tok].ne[1];
    if (g->find("llama.rope.dimension_count")) {
        int32_t n_rot = 0;
        need("llama.rope.dimension_count", &n_rot);
        B200_REQUIRE(n_rot == hp.n_embd_head, "llama_load_gguf: partial rotary dimensions (%d of %d) are not supported", n_rot, hp.n_embd_head);
    }
    b200_llama *c = nullptr;
    rc = b200_llama_new_tp(&hp, device, n_ctx, n_batch, cpu_threads, tp_rank, tp_size, id128, &c);
    if (rc != B200_STATUS_SUCCESS) return rc;
    for (const TensorInfo &t : g->tensors) {
        if (t.name == "rope_freqs.weight") continue;   // the llama builder passes no frequency factors (crates/llama/src/graph_arch.rs:150-165)
        if (t.n_dims > 2 || t.nbytes == 0) {
            b200_llama_free(c);
            B200_REQUIRE(false, "llama_load_gguf: tensor %s has a shape or type this driver does not take", t.name.c_str());
        }
        rc = b200_llama_set_tensor(c, t.name.c_str(), t.type, t.ne[0], t.ne[1], g->map + g->data_offset + t.offset, t.nbytes);
        if (rc != B200_STATUS_SUCCESS) {
            b200_llama_free(c);
            return rc;
        }
    }
    *out = c;
    return B200_STATUS_SUCCESS;
}

int b200_llama_load_gguf(const char *path, int device, int32_t n_ctx, int32_t n_batch, int32_t cpu_threads, b200_llama **out) {
    return b200_llama_load_gguf_tp(path, device, n_ctx, n_batch, cpu_threads, 0, 1, nullptr, out);
}

}  // extern "C"
