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

#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"
#include "llama_b200.h"

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

int tp_comm_init(int rank, int size, const void *id128, void **comm) {
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
void tp_comm_destroy(void *comm) {
    if (comm && g_nccl.CommDestroy) g_nccl.CommDestroy((ncclComm_t)comm);
}
int tp_all_reduce_sum(void *comm, float *buf, size_t count, void *stream) {
    B200_NCCL(g_nccl.AllReduce(buf, buf, count, ncclFloat, ncclSum, (ncclComm_t)comm, (cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}
int tp_all_gather(void *comm, const float *send, float *recv, size_t count_per_rank, void *stream) {
    B200_NCCL(g_nccl.AllGather(send, recv, count_per_rank, ncclFloat, (ncclComm_t)comm, (cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
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
