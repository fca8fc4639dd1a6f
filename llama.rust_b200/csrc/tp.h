// A tensor-parallel group as the backend sees it: this rank's place in it, the NCCL communicator, and the
// peer-memory exchange buffers of the single-kernel collectives (tp_ll.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "llama_b200.h"

namespace b200 {

constexpr int TP_MAX_RANKS = 8;
constexpr int TP_LL_SLOTS = 4;                 // consecutive collectives alternate between slots
constexpr int64_t TP_LL_MAX_ELEMS = 131072;    // largest collective (f32 elements per rank) the exchange buffers carry

// What the exchange kernels get by value.  recv is this rank's buffer, written by every rank (itself included):
// [slot][source rank][element] of 8-byte words (f32 bits, sequence number).  peer[r] is rank r's buffer as mapped
// into this process.  seq counts the collectives run so far and done the CTAs of the current one that have
// finished; both live on the device so that a replayed CUDA graph finds them where the captured launch did.
struct TpExchange {
    unsigned long long *peer[TP_MAX_RANKS];
    unsigned long long *recv;
    unsigned *seq;
    unsigned *done;
    int *err;
    int rank, size;
};

struct TpGroup {
    int rank = 0, size = 1, device = 0;
    void *comm = nullptr;                 // ncclComm_t, null for a group driven through a hook
    b200_tp_hook_fn hook = nullptr;       // tests: the exchange happens on the host
    void *hook_user = nullptr;
    bool ll_ready = false;                // every rank mapped every peer's exchange buffer
    TpExchange x = {};
    void *ll_alloc = nullptr;             // this rank's exchange buffer + counters
    void *peer_mapped[TP_MAX_RANKS] = {nullptr};
    unsigned spin_limit = 0;              // 0 = the default
};

int tp_group_create(int rank, int size, int device, const void *id128, b200_tp_hook_fn hook, void *hook_user, TpGroup **out);
void tp_group_destroy(TpGroup *g);
// in place sum over the ranks of buf[count]; rows x row_len = count.  *capturable is cleared when the call had to
// talk to the host (hook), so that the node list is not captured into a CUDA graph
int tp_all_reduce(TpGroup *g, float *buf, int64_t count, cudaStream_t s, bool *capturable);
// dst[row][r * n_local + j] = rank r's send[row][j]; staging: n_local * size * rows floats of scratch (NCCL path)
int tp_all_gather_rows(TpGroup *g, const float *send, float *dst, int64_t n_local, int64_t rows, float *staging, cudaStream_t s,
                       bool *capturable);

// tp_ll.cu
int launch_tp_ll_all_reduce(const TpExchange &x, float *buf, int64_t count, unsigned spin_limit, cudaStream_t s);
int launch_tp_ll_all_gather(const TpExchange &x, const float *send, float *dst, int64_t n_local, int64_t rows, unsigned spin_limit,
                            cudaStream_t s);
int launch_tp_reorder_gathered(const float *staging, float *dst, int64_t n_local, int64_t rows, int size, cudaStream_t s);

}  // namespace b200
