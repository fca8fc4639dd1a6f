// Row-split tensor parallelism for the decode driver: how a model's tensors are cut across the ranks of one
// node, and the two collectives a sharded layer needs.
//
// The reference has no multi-device path (its scheduler places whole tensors on one backend,
// crates/ggml/src/backend_sched.rs:884-989).  The split here is the usual one for a decoder layer:
//   attn_q / attn_k / attn_v, ffn_gate / ffn_up, output : by output rows (whole heads; FFN rows; vocabulary rows)
//   attn_output, ffn_down                                : by K (the columns that multiply this rank's heads / FFN rows),
//                                                          partial results summed across ranks
//   norms, token_embd                                    : replicated
// so a layer needs one all-reduce after attn_output and one after ffn_down, and the head needs one
// all-gather of the logits.  K is cut on 256-element boundaries, so each rank quantizes its slice of the
// activations to exactly the Q8_K blocks the unsplit row would have; the partial f32 sums are added across
// ranks in NCCL's order instead of the CPU chain's, which is where a tensor-parallel result may differ
// from the single-device one (in the last bits).
//
// NCCL is taken from the process (the copy torch.distributed already loaded) or from libnccl.so.2, at run time:
// the library has no link-time dependency on it, and single-GPU users never touch it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"
#include "llama_b200.h"
#include "tp.h"

using namespace b200;

namespace {

struct Nccl {
    void *lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
Nccl g_nccl;
std::mutex g_nccl_mu;

int nccl_load() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.lib) return B200_STATUS_SUCCESS;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);   // the copy already in the process, if any
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    B200_REQUIRE(h != nullptr, "tensor parallel: cannot load libnccl.so.2 (%s)", dlerror());
    Nccl n;
    n.lib = h;
    *(void **)&n.GetUniqueId = dlsym(h, "ncclGetUniqueId");
    *(void **)&n.CommInitRank = dlsym(h, "ncclCommInitRank");
    *(void **)&n.CommDestroy = dlsym(h, "ncclCommDestroy");
    *(void **)&n.AllReduce = dlsym(h, "ncclAllReduce");
    *(void **)&n.AllGather = dlsym(h, "ncclAllGather");
    *(void **)&n.GetErrorString = dlsym(h, "ncclGetErrorString");
    B200_REQUIRE(n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather && n.GetErrorString,
                 "tensor parallel: libnccl.so.2 lacks a needed symbol");
    g_nccl = n;
    return B200_STATUS_SUCCESS;
}

#define B200_NCCL(call)                                                                         \
    do {                                                                                        \
        ncclResult_t r__ = (call);                                                              \
        if (r__ != ncclSuccess) {                                                               \
            set_error("tensor parallel: %s failed: %s", #call, g_nccl.GetErrorString(r__));     \
            return B200_STATUS_BACKEND_ERROR;                                                   \
        }                                                                                       \
    } while (0)

bool ends_with(const std::string &s, const char *suffix) {
    const size_t n = strlen(suffix);
    return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

size_t block_elems(int type) { return type == B200_TYPE_F32 || type == B200_TYPE_F16 ? 1 : type == B200_TYPE_Q4_K || type == B200_TYPE_Q6_K ? 256 : 32; }
size_t block_bytes(int type) {
    switch (type) {
        case B200_TYPE_F32: return 4;
        case B200_TYPE_F16: return 2;
        case B200_TYPE_Q4_K: return 144;
        case B200_TYPE_Q6_K: return 210;
        case B200_TYPE_Q8_0: return 34;
        case B200_TYPE_Q4_0: return 18;
        case B200_TYPE_MXFP4: return 17;
        default: return 0;
    }
}

}  // namespace

namespace b200 {

// 0 = replicated, 1 = split by rows (ne1), 2 = split by K (ne0)
int tp_split_kind(const char *name) {
    const std::string n(name);
    if (ends_with(n, ".attn_q.weight") || ends_with(n, ".attn_k.weight") || ends_with(n, ".attn_v.weight") ||
        ends_with(n, ".ffn_gate.weight") || ends_with(n, ".ffn_up.weight") || n == "output.weight")
        return 1;
    if (ends_with(n, ".attn_output.weight") || ends_with(n, ".ffn_down.weight")) return 2;
    return 0;
}

static int tp_comm_init(int rank, int size, const void *id128, void **comm) {
    int rc = nccl_load();
    if (rc != B200_STATUS_SUCCESS) return rc;
    ncclUniqueId id;
    static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
    memcpy(&id, id128, sizeof(id));
    ncclComm_t c = nullptr;
    B200_NCCL(g_nccl.CommInitRank(&c, size, id, rank));
    *comm = c;
    return B200_STATUS_SUCCESS;
}

// B200_TP_LL=0 keeps every collective on NCCL (for side-by-side measurements); read once
static bool tp_ll_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_TP_LL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// The exchange buffers of the single-kernel collectives: every rank allocates one receive buffer with cudaMalloc,
// hands its IPC handle round through an NCCL all-gather, and maps every peer's buffer (one process per GPU).
// Whether the group uses them is decided together: one rank that could not map a peer sends everybody to NCCL.
static int tp_exchange_setup(TpGroup *g) {
    const size_t words = (size_t)TP_LL_SLOTS * g->size * (size_t)TP_LL_MAX_ELEMS;
    const size_t bytes = words * 8 + 256;
    int ok = 1;
    if (!tp_ll_enabled() || cudaMalloc(&g->ll_alloc, bytes) != cudaSuccess) {
        cudaGetLastError();
        g->ll_alloc = nullptr;
        ok = 0;
    }
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (ok && (cudaMemset(g->ll_alloc, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&mine, g->ll_alloc) != cudaSuccess)) {
        cudaGetLastError();
        ok = 0;
    }
    // handles (64 bytes each) and the ranks' verdicts travel through the communicator
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
    uint8_t *dev = nullptr;
    B200_CUDA(cudaMalloc((void **)&dev, (size_t)64 * g->size + 64));
    int *dev_ok = (int *)(dev + (size_t)64 * g->size);
    B200_CUDA(cudaMemcpy(dev + (size_t)64 * g->rank, &mine, 64, cudaMemcpyHostToDevice));
    cudaStream_t s = nullptr;
    auto gather_handles = [&]() -> int {
        B200_NCCL(g_nccl.AllGather(dev + (size_t)64 * g->rank, dev, 64, ncclChar, (ncclComm_t)g->comm, s));
        B200_CUDA(cudaStreamSynchronize(s));
        return B200_STATUS_SUCCESS;
    };
    int rc = gather_handles();
    if (rc != B200_STATUS_SUCCESS) { cudaFree(dev); return rc; }
    std::string handles((size_t)64 * g->size, '\0');
    B200_CUDA(cudaMemcpy(&handles[0], dev, handles.size(), cudaMemcpyDeviceToHost));
    for (int r = 0; r < g->size && ok; r++) {
        if (r == g->rank) { g->peer_mapped[r] = nullptr; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, &handles[(size_t)64 * r], 64);
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = 0;
        } else {
            g->peer_mapped[r] = p;
        }
    }
    B200_CUDA(cudaMemcpy(dev_ok, &ok, sizeof(int), cudaMemcpyHostToDevice));
    auto agree = [&]() -> int {
        B200_NCCL(g_nccl.AllReduce(dev_ok, dev_ok, 1, ncclInt, ncclMin, (ncclComm_t)g->comm, s));
        B200_CUDA(cudaStreamSynchronize(s));
        return B200_STATUS_SUCCESS;
    };
    rc = agree();
    if (rc != B200_STATUS_SUCCESS) { cudaFree(dev); return rc; }
    int all_ok = 0;
    B200_CUDA(cudaMemcpy(&all_ok, dev_ok, sizeof(int), cudaMemcpyDeviceToHost));
    cudaFree(dev);
    g->ll_ready = all_ok == 1;
    if (!g->ll_ready) return B200_STATUS_SUCCESS;   // NCCL serves every collective
    TpExchange &x = g->x;
    x.rank = g->rank;
    x.size = g->size;
    x.recv = (unsigned long long *)g->ll_alloc;
    for (int r = 0; r < g->size; r++) x.peer[r] = r == g->rank ? x.recv : (unsigned long long *)g->peer_mapped[r];
    x.seq = (unsigned *)((uint8_t *)g->ll_alloc + words * 8);
    x.done = x.seq + 1;
    return device_error_word(&x.err);
}

int tp_group_create(int rank, int size, int device, const void *id128, b200_tp_hook_fn hook, void *hook_user, TpGroup **out) {
    *out = nullptr;
    B200_REQUIRE(size >= 2 && size <= TP_MAX_RANKS && rank >= 0 && rank < size, "tensor parallel: rank %d of %d (2 to %d ranks)", rank, size,
                 TP_MAX_RANKS);
    B200_REQUIRE(hook != nullptr || id128 != nullptr, "tensor parallel: a group needs the shared id (or an exchange hook)");
    B200_CUDA(cudaSetDevice(device));
    TpGroup *g = new TpGroup();
    g->rank = rank;
    g->size = size;
    g->device = device;
    g->hook = hook;
    g->hook_user = hook_user;
    if (!hook) {
        int rc = tp_comm_init(rank, size, id128, &g->comm);
        if (rc == B200_STATUS_SUCCESS) rc = tp_exchange_setup(g);
        if (rc != B200_STATUS_SUCCESS) { tp_group_destroy(g); return rc; }
    }
    *out = g;
    return B200_STATUS_SUCCESS;
}

void tp_group_destroy(TpGroup *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < TP_MAX_RANKS; r++)
        if (g->peer_mapped[r]) cudaIpcCloseMemHandle(g->peer_mapped[r]);
    if (g->comm && g_nccl.CommDestroy) g_nccl.CommDestroy((ncclComm_t)g->comm);   // peers may still be writing until here
    if (g->ll_alloc) cudaFree(g->ll_alloc);
    cudaGetLastError();
    delete g;
}

int tp_all_reduce(TpGroup *g, float *buf, int64_t count, cudaStream_t s, bool *capturable) {
    B200_REQUIRE(g != nullptr, "tensor parallel: no group attached to this backend");
    if (count == 0) return B200_STATUS_SUCCESS;
    if (g->hook) {
        if (capturable) *capturable = false;
        B200_CUDA(cudaStreamSynchronize(s));
        const int rc = g->hook(g->hook_user, 0, g->rank, g->size, buf, count, nullptr, 0, 0);
        B200_REQUIRE(rc == 0, "tensor parallel: the exchange hook failed (%d)", rc);
        return B200_STATUS_SUCCESS;
    }
    if (g->ll_ready && count <= TP_LL_MAX_ELEMS) return launch_tp_ll_all_reduce(g->x, buf, count, g->spin_limit, s);
    B200_NCCL(g_nccl.AllReduce(buf, buf, (size_t)count, ncclFloat, ncclSum, (ncclComm_t)g->comm, s));
    return B200_STATUS_SUCCESS;
}

int tp_all_gather_rows(TpGroup *g, const float *send, float *dst, int64_t n_local, int64_t rows, float *staging, cudaStream_t s,
                       bool *capturable) {
    B200_REQUIRE(g != nullptr, "tensor parallel: no group attached to this backend");
    if (n_local * rows == 0) return B200_STATUS_SUCCESS;
    if (g->hook) {
        if (capturable) *capturable = false;
        B200_CUDA(cudaStreamSynchronize(s));
        const int rc = g->hook(g->hook_user, 1, g->rank, g->size, const_cast<float *>(send), n_local * rows, dst, n_local, rows);
        B200_REQUIRE(rc == 0, "tensor parallel: the exchange hook failed (%d)", rc);
        return B200_STATUS_SUCCESS;
    }
    if (g->ll_ready && n_local * rows <= TP_LL_MAX_ELEMS) return launch_tp_ll_all_gather(g->x, send, dst, n_local, rows, g->spin_limit, s);
    if (rows == 1) {   // the ranks' slices side by side are the whole row
        B200_NCCL(g_nccl.AllGather(send, dst, (size_t)n_local, ncclFloat, (ncclComm_t)g->comm, s));
        return B200_STATUS_SUCCESS;
    }
    B200_REQUIRE(staging != nullptr, "tensor parallel: all-gather of %lld rows needs a staging block", (long long)rows);
    B200_NCCL(g_nccl.AllGather(send, staging, (size_t)(n_local * rows), ncclFloat, (ncclComm_t)g->comm, s));
    return launch_tp_reorder_gathered(staging, dst, n_local, rows, g->size, s);
}

}  // namespace b200

extern "C" {

int b200_tp_unique_id(void *id128) {
    B200_REQUIRE(id128 != nullptr, "tp_unique_id: null argument");
    int rc = nccl_load();
    if (rc != B200_STATUS_SUCCESS) return rc;
    ncclUniqueId id;
    B200_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id128, &id, sizeof(id));
    return B200_STATUS_SUCCESS;
}

int b200_tp_shard_shape(const char *name, int type, int64_t ne0, int64_t ne1, int32_t tp_size, int32_t *split, int64_t *ne0_local,
                        int64_t *ne1_local) {
    B200_REQUIRE(name && split && ne0_local && ne1_local, "tp_shard_shape: null argument");
    B200_REQUIRE(tp_size >= 1, "tp_shard_shape: tp_size %d", tp_size);
    const int kind = tp_size == 1 ? 0 : tp_split_kind(name);
    *split = kind;
    *ne0_local = ne0;
    *ne1_local = ne1;
    if (kind == 1) {
        B200_REQUIRE(ne1 % tp_size == 0 && (ne1 / tp_size) % TILE_ROWS == 0, "%s: %lld rows do not split into %d shards of whole 32-row tiles",
                     name, (long long)ne1, tp_size);
        *ne1_local = ne1 / tp_size;
    } else if (kind == 2) {
        const int64_t cut = is_quant_type(type) ? GROUP_K : 1;
        B200_REQUIRE(ne0 % tp_size == 0 && (ne0 / tp_size) % cut == 0, "%s: k = %lld does not split into %d shards on 256-element boundaries",
                     name, (long long)ne0, tp_size);
        *ne0_local = ne0 / tp_size;
    }
    return B200_STATUS_SUCCESS;
}

int b200_tp_shard_tensor(const char *name, int type, int64_t ne0, int64_t ne1, const void *data, int32_t tp_rank, int32_t tp_size,
                         void *out, size_t out_nbytes) {
    B200_REQUIRE(data != nullptr && out != nullptr, "tp_shard_tensor: null argument");
    B200_REQUIRE(tp_rank >= 0 && tp_rank < tp_size, "tp_shard_tensor: rank %d of %d", tp_rank, tp_size);
    int32_t split = 0;
    int64_t l0 = 0, l1 = 0;
    int rc = b200_tp_shard_shape(name, type, ne0, ne1, tp_size, &split, &l0, &l1);
    if (rc != B200_STATUS_SUCCESS) return rc;
    const size_t be = block_elems(type), bb = block_bytes(type);
    B200_REQUIRE(bb != 0 && ne0 % be == 0, "tp_shard_tensor: %s: unsupported type %d or row length %lld", name, type, (long long)ne0);
    const size_t row = ne0 / be * bb, row_local = l0 / be * bb;
    B200_REQUIRE(out_nbytes == row_local * (size_t)l1, "tp_shard_tensor: %s: %zu bytes given for the shard, %zu expected", name, out_nbytes,
                 row_local * (size_t)l1);
    const uint8_t *src = (const uint8_t *)data;
    uint8_t *dst = (uint8_t *)out;
    if (split == 0) {
        memcpy(dst, src, row * ne1);
    } else if (split == 1) {
        memcpy(dst, src + (size_t)tp_rank * l1 * row, row * l1);
    } else {
        for (int64_t r = 0; r < ne1; r++) memcpy(dst + r * row_local, src + r * row + (size_t)tp_rank * row_local, row_local);
    }
    return B200_STATUS_SUCCESS;
}

}  // extern "C"
