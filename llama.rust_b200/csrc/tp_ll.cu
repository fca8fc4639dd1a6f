// Single-kernel collectives of a tensor-parallel group over peer-mapped memory (NVLink / NVSwitch).
//
// A decode step all-reduces one row of d_model floats after attn_output and after ffn_down of every layer:
// 16 to 32 KB, 160 times per token on an 80-layer model.  At that size a collective is all latency, so it is
// one small kernel with no host involvement and no library call:
//   * every thread takes one element; it stores (value, sequence number) as ONE naturally aligned 8-byte word
//     into the receive buffer of every rank of the group (plain st.global over NVLink, its own buffer included);
//     an 8-byte scalar store is single-copy atomic, so the word itself tells the reader that the value has
//     arrived: no separate flag, no fence between data and flag;
//   * it then polls its element's word from every source rank in its OWN receive buffer until the sequence
//     number matches, and adds the values in rank order ((p0 + p1) + p2 ..., each add rounded to f32): every rank
//     computes the same bits, and a CPU restatement of the cut reproduces them exactly;
//   * the sequence number comes from a counter on the device (a captured CUDA graph replays the same launch);
//     the last CTA to finish advances it.  Consecutive collectives use different slots of the buffer, so a fast
//     rank that has already moved on to the next collective does not overwrite what a slow one still reads
//     (a rank can be at most one collective ahead: it needs every peer's words of the current one to go on).
// Every poll is bounded; on expiry the thread records code 4 in the device's error word and leaves its output
// element unwritten.  No multicast of any kind is involved: loads are local, stores are per-peer.
#include "common.cuh"
#include "tp.h"

namespace b200 {

namespace {

constexpr unsigned TP_SPIN_DEFAULT = 1u << 23;   // polls with a short sleep between them: several seconds in all

__device__ __forceinline__ unsigned long long ld_word(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_word(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_counter(const unsigned *p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// word e of source rank r in slot `slot` of a receive buffer
__device__ __forceinline__ size_t word_index(unsigned slot, int size, int r, int64_t e) {
    return ((size_t)slot * size + r) * (size_t)TP_LL_MAX_ELEMS + (size_t)e;
}

// stores w as this rank's word e of the current slot in every rank's receive buffer
__device__ __forceinline__ void push_word(const TpExchange &x, unsigned slot, int64_t e, unsigned long long w) {
    const size_t at = word_index(slot, x.size, x.rank, e);
#pragma unroll
    for (int r = 0; r < TP_MAX_RANKS; r++)   // constant indices: the pointer table stays in the parameter bank
        if (r < x.size) st_word(x.peer[r] + at, w);
}

// waits (bounded) for source rank r's word e of sequence number seq; false on expiry
__device__ __forceinline__ bool poll_word(const TpExchange &x, unsigned slot, int r, int64_t e, unsigned seq, unsigned limit, float *v) {
    const unsigned long long *src = x.recv + word_index(slot, x.size, r, e);
    for (unsigned n = 0; n < limit; n++) {
        const unsigned long long got = ld_word(src);
        if ((unsigned)(got >> 32) == seq) {
            *v = __uint_as_float((unsigned)got);
            return true;
        }
        if (n > 32) __nanosleep(n > 4096 ? 512 : 64);
    }
    return false;
}

// the last CTA of a collective to get here advances the sequence counter (every CTA read it when it started)
__device__ __forceinline__ void finish_collective(const TpExchange &x, bool bad) {
    if (bad) atomicExch(x.err, 4);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(x.done, 1u) == gridDim.x - 1) {
            atomicExch(x.done, 0u);
            __threadfence();
            atomicAdd(x.seq, 1u);
        }
    }
}

__global__ void __launch_bounds__(256)
tp_ll_all_reduce_kernel(TpExchange x, float *buf, int64_t count, unsigned limit) {
    pdl_trigger();
    pdl_wait();   // buf is the previous kernel's output; the counter was advanced by the previous collective
    const unsigned seq = ld_counter(x.seq) + 1u;
    const unsigned slot = seq % TP_LL_SLOTS;
    const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
    bool bad = false;
    if (e < count) {
        push_word(x, slot, e, ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(buf[e]));
        float sum = 0.0f;
        for (int r = 0; r < x.size && !bad; r++) {
            float v;
            if (!poll_word(x, slot, r, e, seq, limit, &v)) bad = true;
            else sum = r == 0 ? v : __fadd_rn(sum, v);
        }
        if (!bad) buf[e] = sum;
    }
    finish_collective(x, bad);
}

// dst[row][r * n_local + j] = rank r's send[row][j]
__global__ void __launch_bounds__(256)
tp_ll_all_gather_kernel(TpExchange x, const float *send, float *dst, int64_t n_local, int64_t rows, unsigned limit) {
    pdl_trigger();
    pdl_wait();
    const unsigned seq = ld_counter(x.seq) + 1u;
    const unsigned slot = seq % TP_LL_SLOTS;
    const int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x;
    bool bad = false;
    if (e < n_local * rows) {
        push_word(x, slot, e, ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(send[e]));
        const int64_t row = e / n_local, j = e - row * n_local;
        for (int r = 0; r < x.size && !bad; r++) {
            float v;
            if (!poll_word(x, slot, r, e, seq, limit, &v)) bad = true;
            else dst[row * n_local * x.size + (int64_t)r * n_local + j] = v;
        }
    }
    finish_collective(x, bad);
}

// NCCL's all-gather leaves [rank][row][j]; the logits are wanted as [row][rank][j]
__global__ void __launch_bounds__(256)
tp_reorder_gathered_kernel(const float *staging, float *dst, int64_t n_local, int64_t rows, int size) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n_local * rows * size) return;
    const int64_t r = i / (n_local * rows), rest = i - r * n_local * rows, row = rest / n_local, j = rest - row * n_local;
    dst[row * n_local * size + r * n_local + j] = staging[i];
}

}  // namespace

int launch_tp_ll_all_reduce(const TpExchange &x, float *buf, int64_t count, unsigned spin_limit, cudaStream_t s) {
    B200_REQUIRE(count > 0 && count <= TP_LL_MAX_ELEMS, "tp all-reduce: %lld elements exceed the exchange buffer", (long long)count);
    return launch_pdl(tp_ll_all_reduce_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, s, x, buf, count,
                      spin_limit ? spin_limit : TP_SPIN_DEFAULT);
}

int launch_tp_ll_all_gather(const TpExchange &x, const float *send, float *dst, int64_t n_local, int64_t rows, unsigned spin_limit,
                            cudaStream_t s) {
    const int64_t count = n_local * rows;
    B200_REQUIRE(count > 0 && count <= TP_LL_MAX_ELEMS, "tp all-gather: %lld elements exceed the exchange buffer", (long long)count);
    return launch_pdl(tp_ll_all_gather_kernel, dim3((unsigned)((count + 255) / 256)), dim3(256), 0, s, x, send, dst, n_local, rows,
                      spin_limit ? spin_limit : TP_SPIN_DEFAULT);
}

int launch_tp_reorder_gathered(const float *staging, float *dst, int64_t n_local, int64_t rows, int size, cudaStream_t s) {
    const int64_t total = n_local * rows * size;
    if (total == 0) return B200_STATUS_SUCCESS;
    return launch_pdl(tp_reorder_gathered_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, staging, dst, n_local, rows, size);
}

}  // namespace b200
