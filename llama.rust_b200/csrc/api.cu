// Op-level C entry points of libggml-b200 (declared in include/ggml_b200.h).
// Argument checking, scratch management and route selection live here; the
// kernels are in the other translation units.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace b200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what, const char *file, int line) {
    set_error("CUDA error %d (%s) at %s:%d: %s", (int)e, cudaGetErrorString(e), file, line, what);
    if (e == cudaErrorMemoryAllocation) return B200_STATUS_ALLOC_FAILED;
    return B200_STATUS_BACKEND_ERROR;
}

// Numerics policy of the library: 1 = fast (tolerance-mode kernels where they exist: f32-accumulating attention,
// ...), 0 = exact (every kernel reproduces the reference CPU route's arithmetic bit for bit).  B200_NUMERICS=exact|fast
// sets the start value (fast when unset); b200_set_numerics changes it at run time.
static int g_numerics = -1;
int numerics_mode() {
    if (g_numerics < 0) {
        const char *e = getenv("B200_NUMERICS");
        g_numerics = (e && (e[0] == 'e' || e[0] == 'E' || e[0] == '0')) ? 0 : 1;
    }
    return g_numerics;
}
void set_numerics_mode(int mode) { g_numerics = mode ? 1 : 0; }

bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// ---- scratch: one growing allocation per device ------------------------------
struct Scratch {
    void *ptr = nullptr;
    size_t bytes = 0;
};
static std::mutex g_scratch_mu;
static unsigned long long g_alloc_count = 0;
static thread_local int g_no_scratch = 0;
NoScratchScope::NoScratchScope() { g_no_scratch++; }
NoScratchScope::~NoScratchScope() { g_no_scratch--; }
bool no_scratch_mode() { return g_no_scratch > 0; }
unsigned long long library_alloc_count() {
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    return g_alloc_count;
}
static Scratch g_scratch[4][64];   // [0] general scratch, [1] the K-split exchange of the decode mat-mul (lives across the other's users)
static unsigned long long g_scratch_gen = 0;

// bumped whenever a scratch block is replaced: a captured CUDA graph that baked the old address in is stale
unsigned long long scratch_generation() {
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    return g_scratch_gen;
}

static int scratch_get_slot(int slot, size_t bytes, void **ptr);
int scratch_get(size_t bytes, void **ptr) { return scratch_get_slot(0, bytes, ptr); }
int scratch_get_kx(size_t bytes, void **ptr) { return scratch_get_slot(1, bytes, ptr); }
int scratch_get_lists(size_t bytes, void **ptr) { return scratch_get_slot(2, bytes, ptr); }   // attention's visible-position lists
int scratch_get_images(size_t bytes, void **ptr) { return scratch_get_slot(3, bytes, ptr); }  // the prompt mat-mul's f16 operand images
static int scratch_get_slot(int slot, size_t bytes, void **ptr) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "scratch: device index %d out of range", dev);
    B200_REQUIRE(!no_scratch_mode(), "a route that needs library scratch (%zu bytes, block %d) was taken inside an entry point that may not allocate",
                 bytes, slot);
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch &s = g_scratch[slot][dev];
    if (s.bytes < bytes) {
        if (s.ptr) {
            // work queued on any stream may still read the old block
            B200_CUDA(cudaDeviceSynchronize());
            B200_CUDA(cudaFree(s.ptr));
            s.ptr = nullptr;
            s.bytes = 0;
        }
        size_t want = bytes + bytes / 4;
        if (want < (size_t)(slot == 0 ? 8 : 2) << 20) want = (size_t)(slot == 0 ? 8 : 2) << 20;
        B200_CUDA(cudaMalloc(&s.ptr, want));
        s.bytes = want;
        g_scratch_gen++;
        g_alloc_count++;
    }
    *ptr = s.ptr;
    return B200_STATUS_SUCCESS;
}

// What the reference picks for (type, n, m): crates/ggml/src/compute.rs:1420-1841.
int pick_route(int type, int64_t n, int64_t m) {
    switch (type) {
        case B200_TYPE_Q4_K:
            if (n % 8 == 0) return B200_ROUTE_REPACK;
            return m >= 8 ? B200_ROUTE_TILED : B200_ROUTE_ROWDOT;
        case B200_TYPE_Q6_K: return m >= 8 ? B200_ROUTE_TILED : B200_ROUTE_ROWDOT;
        case B200_TYPE_Q8_0: return B200_ROUTE_ROWDOT;
        case B200_TYPE_Q4_0:
        case B200_TYPE_MXFP4: return n % 8 == 0 ? B200_ROUTE_REPACK : B200_ROUTE_ROWDOT;
        default: return -1;
    }
}

// which activation quantizer a (type, route) reads
int act_kind_for(int type, int route, int64_t m) {
    if (!is_k_quant(type)) return B200_ACT_Q8_0;
    // the Q4_K 8x8 route quantizes whole groups of 4 rows with the 4x8 rule (compute.rs:5322-5400)
    if (type == B200_TYPE_Q4_K && route == B200_ROUTE_REPACK && m >= 4) return B200_ACT_Q8_K_MIXED;
    return B200_ACT_Q8_K;
}

static size_t ggml_row_bytes(int type, int64_t k) { return (size_t)(k / GROUP_K) * group_src_bytes(type); }

}  // namespace b200

using namespace b200;

extern "C" {

const char *b200_last_error(void) { return g_err; }

int b200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int b200_set_device(int device) {
    B200_CUDA(cudaSetDevice(device));
    return B200_STATUS_SUCCESS;
}

int b200_device_info(int device, char *name, size_t name_len, size_t *free_bytes, size_t *total_bytes, int *sm_count,
                     int *cc_major, int *cc_minor) {
    cudaDeviceProp p;
    B200_CUDA(cudaGetDeviceProperties(&p, device));
    if (name && name_len) snprintf(name, name_len, "%s", p.name);
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    if (free_bytes || total_bytes) {
        int cur = 0;
        B200_CUDA(cudaGetDevice(&cur));
        B200_CUDA(cudaSetDevice(device));
        size_t f = 0, t = 0;
        cudaError_t e = cudaMemGetInfo(&f, &t);
        cudaSetDevice(cur);
        B200_CUDA(e);
        if (free_bytes) *free_bytes = f;
        if (total_bytes) *total_bytes = t;
    }
    return B200_STATUS_SUCCESS;
}

int b200_synchronize(void *stream) {
    B200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}

int b200_kernel_error(int *code) {
    B200_REQUIRE(code != nullptr, "kernel_error: null out pointer");
    return gemv_stream_error(code);
}

void b200_set_numerics(int mode) { set_numerics_mode(mode); }
int b200_get_numerics(void) { return numerics_mode(); }

unsigned long long b200_debug_alloc_count(void) { return library_alloc_count(); }

void b200_debug_stream_wait(int spin_limit, int skip_unit) { gemv_stream_debug_wait(spin_limit, skip_unit); }
unsigned long long b200_debug_decode_step_launches(void) { return decode_persistent_launches(); }
int b200_debug_fa_prefill_profile(unsigned long long *out, int n) { return flash_attn_prefill_profile(out, n); }
int b200_debug_gemm_fast_profile(unsigned long long *out, int n) { return gemm_fast_profile(out, n); }
void b200_debug_gemm_fast_wait(int spin_limit, int mute_cta) { gemm_fast_debug_wait(spin_limit, mute_cta); }
void b200_debug_rows_ring_wait(int spin_limit, int skip_unit) { gemm_rows_ring_debug_wait(spin_limit, skip_unit); }
int b200_debug_decode_step_times(unsigned long long *out, int n) { return decode_persistent_times(out, n); }
void b200_debug_decode_step_wait(int spin_limit, int skip_cta, int skip_barrier) { decode_persistent_debug(spin_limit, skip_cta, skip_barrier); }

int b200_prompt_kernel_choice(int64_t n, int64_t m, int sm_count) { return gemm_chain_pick_for(n, m, sm_count); }

int b200_malloc(void **dev_ptr, size_t bytes) {
    B200_REQUIRE(dev_ptr != nullptr, "malloc: null out pointer");
    *dev_ptr = nullptr;
    if (bytes == 0) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaMalloc(dev_ptr, bytes));
    return B200_STATUS_SUCCESS;
}

int b200_free(void *dev_ptr) {
    if (dev_ptr) B200_CUDA(cudaFree(dev_ptr));
    return B200_STATUS_SUCCESS;
}

int b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}

int b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    B200_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}

int b200_memset(void *dst, int value, size_t bytes, void *stream) {
    if (bytes == 0) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}

int b200_host_alloc_pinned(void **host_ptr, size_t bytes) {
    B200_REQUIRE(host_ptr != nullptr, "host_alloc_pinned: null out pointer");
    B200_CUDA(cudaMallocHost(host_ptr, bytes));
    return B200_STATUS_SUCCESS;
}

int b200_host_free_pinned(void *host_ptr) {
    if (host_ptr) B200_CUDA(cudaFreeHost(host_ptr));
    return B200_STATUS_SUCCESS;
}

size_t b200_weight_nbytes(int type, int64_t n_rows, int64_t k) {
    if (!is_quant_type(type) || n_rows < 0 || k <= 0 || k % GROUP_K != 0) return 0;
    const int64_t tiles = (n_rows + TILE_ROWS - 1) / TILE_ROWS;
    return (size_t)tiles * (size_t)(k / GROUP_K) * (size_t)chunk_bytes(type);
}

// Uploads in pieces of whole row tiles so that the staging copy stays small.
int b200_weight_upload(int type, int64_t n_rows, int64_t k, const void *host_blocks, void *dev_tiles, void *stream) {
    B200_REQUIRE(is_quant_type(type), "weight_upload: type %d is not a supported quantized type", type);
    B200_REQUIRE(k > 0 && k % GROUP_K == 0, "weight_upload: k = %lld must be a positive multiple of 256", (long long)k);
    B200_REQUIRE(n_rows >= 0, "weight_upload: negative row count");
    if (n_rows == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(host_blocks && dev_tiles, "weight_upload: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t rb = ggml_row_bytes(type, k);
    const int64_t groups = k / GROUP_K;
    int64_t rows_per_piece = ((int64_t)(64 << 20) / (int64_t)rb) / TILE_ROWS * TILE_ROWS;
    if (rows_per_piece < TILE_ROWS) rows_per_piece = TILE_ROWS;
    void *stage = nullptr;
    B200_CUDA(cudaMalloc(&stage, (size_t)std::min<int64_t>(rows_per_piece, n_rows) * rb));
    int rc = B200_STATUS_SUCCESS;
    for (int64_t r0 = 0; r0 < n_rows && rc == B200_STATUS_SUCCESS; r0 += rows_per_piece) {
        const int64_t nr = std::min<int64_t>(rows_per_piece, n_rows - r0);
        cudaError_t e = cudaMemcpyAsync(stage, (const uint8_t *)host_blocks + (size_t)r0 * rb, (size_t)nr * rb,
                                        cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) { rc = cuda_fail(e, "cudaMemcpyAsync(stage)", __FILE__, __LINE__); break; }
        uint8_t *dst = (uint8_t *)dev_tiles + (size_t)(r0 / TILE_ROWS) * groups * chunk_bytes(type);
        rc = launch_repack(type, nr, k, (const uint8_t *)stage, dst, false, s);
        if (rc == B200_STATUS_SUCCESS) {
            e = cudaStreamSynchronize(s);
            if (e != cudaSuccess) rc = cuda_fail(e, "cudaStreamSynchronize", __FILE__, __LINE__);
        }
    }
    cudaFree(stage);
    return rc;
}

int b200_weight_download(int type, int64_t n_rows, int64_t k, const void *dev_tiles, void *host_blocks, void *stream) {
    B200_REQUIRE(is_quant_type(type), "weight_download: type %d is not a supported quantized type", type);
    B200_REQUIRE(k > 0 && k % GROUP_K == 0, "weight_download: k = %lld must be a positive multiple of 256", (long long)k);
    if (n_rows <= 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(host_blocks && dev_tiles, "weight_download: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t rb = ggml_row_bytes(type, k);
    const int64_t groups = k / GROUP_K;
    int64_t rows_per_piece = ((int64_t)(64 << 20) / (int64_t)rb) / TILE_ROWS * TILE_ROWS;
    if (rows_per_piece < TILE_ROWS) rows_per_piece = TILE_ROWS;
    void *stage = nullptr;
    B200_CUDA(cudaMalloc(&stage, (size_t)std::min<int64_t>(rows_per_piece, n_rows) * rb));
    int rc = B200_STATUS_SUCCESS;
    for (int64_t r0 = 0; r0 < n_rows && rc == B200_STATUS_SUCCESS; r0 += rows_per_piece) {
        const int64_t nr = std::min<int64_t>(rows_per_piece, n_rows - r0);
        const uint8_t *src = (const uint8_t *)dev_tiles + (size_t)(r0 / TILE_ROWS) * groups * chunk_bytes(type);
        rc = launch_repack(type, nr, k, src, (uint8_t *)stage, true, s);
        if (rc != B200_STATUS_SUCCESS) break;
        cudaError_t e = cudaMemcpyAsync((uint8_t *)host_blocks + (size_t)r0 * rb, stage, (size_t)nr * rb,
                                        cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) rc = cuda_fail(e, "download copy", __FILE__, __LINE__);
    }
    cudaFree(stage);
    return rc;
}

int b200_dequantize(int type, int64_t n_rows, int64_t k, const void *dev_tiles, float *dev_out, void *stream) {
    return launch_dequantize(type, n_rows, k, (const uint8_t *)dev_tiles, dev_out, (cudaStream_t)stream);
}

int b200_quantize_activations(int kind, int64_t m, int64_t k, const float *dev_x, void *host_blocks, void *stream) {
    B200_REQUIRE(m >= 0 && k > 0, "quantize_activations: bad shape m=%lld k=%lld", (long long)m, (long long)k);
    B200_REQUIRE(kind != B200_ACT_Q8_K_4X8 || m % 4 == 0, "quantize_activations: the 4x8 form needs m %% 4 == 0");
    if (m == 0) return B200_STATUS_SUCCESS;
    cudaStream_t s = (cudaStream_t)stream;
    void *scratch = nullptr;
    int rc = scratch_get(act_scratch_bytes(m, k), &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    ActBuf a = act_carve(scratch, m, k);
    rc = launch_quantize_acts(kind, m, k, dev_x, k, a, s);
    if (rc != B200_STATUS_SUCCESS) return rc;
    std::vector<int8_t> qs((size_t)m * k);
    B200_CUDA(cudaMemcpyAsync(qs.data(), a.qs, qs.size(), cudaMemcpyDeviceToHost, s));
    uint8_t *out = (uint8_t *)host_blocks;
    if (kind == B200_ACT_Q8_0) {
        const int64_t nb = k / 32;
        std::vector<uint16_t> dh((size_t)m * nb);
        B200_CUDA(cudaMemcpyAsync(dh.data(), a.dh, dh.size() * 2, cudaMemcpyDeviceToHost, s));
        B200_CUDA(cudaStreamSynchronize(s));
        for (int64_t r = 0; r < m; r++)
            for (int64_t b = 0; b < nb; b++) {
                uint8_t *blk = out + (r * nb + b) * 34;
                memcpy(blk, &dh[r * nb + b], 2);
                memcpy(blk + 2, &qs[r * k + b * 32], 32);
            }
        return B200_STATUS_SUCCESS;
    }
    const int64_t nb = k / 256;
    std::vector<float> d((size_t)m * nb);
    std::vector<int16_t> bs((size_t)m * (k / 16));
    B200_CUDA(cudaMemcpyAsync(d.data(), a.d, d.size() * 4, cudaMemcpyDeviceToHost, s));
    B200_CUDA(cudaMemcpyAsync(bs.data(), a.bsums, bs.size() * 2, cudaMemcpyDeviceToHost, s));
    B200_CUDA(cudaStreamSynchronize(s));
    if (kind == B200_ACT_Q8_K) {
        for (int64_t r = 0; r < m; r++)
            for (int64_t b = 0; b < nb; b++) {
                uint8_t *blk = out + (r * nb + b) * 292;
                memcpy(blk, &d[r * nb + b], 4);
                memcpy(blk + 4, &qs[r * k + b * 256], 256);
                memcpy(blk + 260, &bs[r * (k / 16) + b * 16], 32);
            }
    } else {  // block_q8_Kx4: crates/ggml/src/repack.rs:1557-1606
        for (int64_t g = 0; g < m / 4; g++)
            for (int64_t b = 0; b < nb; b++) {
                uint8_t *blk = out + (g * nb + b) * 1168;
                int16_t *obs = (int16_t *)(blk + 1040);
                for (int r = 0; r < 4; r++) {
                    const int64_t row = g * 4 + r;
                    memcpy(blk + 4 * r, &d[row * nb + b], 4);
                    for (int el = 0; el < 256; el++)
                        blk[16 + (el / 8) * 32 + r * 8 + el % 8] = (uint8_t)qs[row * k + b * 256 + el];
                    for (int j = 0; j < 16; j++) obs[16 * (j / 4) + 4 * r + j % 4] = bs[row * (k / 16) + b * 16 + j];
                }
            }
    }
    return B200_STATUS_SUCCESS;
}

size_t b200_act_scratch_nbytes(int64_t m, int64_t k) {
    if (m < 0 || k <= 0 || k % 32 != 0) return 0;
    return act_scratch_bytes(m, k);
}

int b200_quantize_activations_device(int kind, int64_t m, int64_t k, const float *dev_x, int64_t ldx, void *dev_act,
                                     void *stream) {
    B200_REQUIRE(m >= 0 && k > 0 && ldx >= k, "quantize_activations_device: bad shape");
    if (m == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_x && dev_act, "quantize_activations_device: null pointer");
    B200_REQUIRE(((uintptr_t)dev_act & 255) == 0, "quantize_activations_device: scratch must be 256-byte aligned");
    return launch_quantize_acts(kind, m, k, dev_x, ldx, act_carve(dev_act, m, k), (cudaStream_t)stream);
}

int b200_event_create(void **event) {
    B200_REQUIRE(event != nullptr, "event_create: null out pointer");
    cudaEvent_t e;
    B200_CUDA(cudaEventCreate(&e));
    *event = (void *)e;
    return B200_STATUS_SUCCESS;
}
int b200_event_destroy(void *event) {
    if (event) B200_CUDA(cudaEventDestroy((cudaEvent_t)event));
    return B200_STATUS_SUCCESS;
}
int b200_event_record(void *event, void *stream) {
    B200_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
    return B200_STATUS_SUCCESS;
}
int b200_event_synchronize(void *event) {
    B200_CUDA(cudaEventSynchronize((cudaEvent_t)event));
    return B200_STATUS_SUCCESS;
}
int b200_event_elapsed_ms(void *start, void *stop, float *ms) {
    B200_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return B200_STATUS_SUCCESS;
}

static int check_mul_mat_args(int type, int64_t n, int64_t k, int64_t m) {
    B200_REQUIRE(is_quant_type(type), "mul_mat: weight type %d is not supported", type);
    B200_REQUIRE(n >= 0 && m >= 0 && k > 0, "mul_mat: bad shape n=%lld k=%lld m=%lld", (long long)n, (long long)k,
                 (long long)m);
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat: k = %lld must be a multiple of 256", (long long)k);
    return B200_STATUS_SUCCESS;
}

int b200_mul_mat_q8(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const void *dev_act, int act_kind,
                    float *dev_dst, int64_t lddst, int route, void *stream) {
    int rc = check_mul_mat_args(type, n, k, m);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_w && dev_act && dev_dst, "mul_mat_q8: null pointer");
    B200_REQUIRE(lddst >= n, "mul_mat_q8: dst row stride smaller than n");
    if (route == B200_ROUTE_AUTO) route = pick_route(type, n, m);
    B200_REQUIRE(act_kind == act_kind_for(type, route, m), "mul_mat_q8: activation kind %d does not fit type %d", act_kind,
                 type);
    ActBuf a = act_carve(const_cast<void *>(dev_act), m, k);
    return launch_gemv(type, route, n, k, m, (const uint8_t *)dev_w, a.view(), dev_dst, lddst, (cudaStream_t)stream);
}

// Times `reps` back-to-back launches of b200_mul_mat_q8 that rotate over n_w copies of the weights, as one replayed
// CUDA graph: what a kernel costs inside a decode step, where a captured graph issues the launches and no host
// call sits between them.  *us_per_launch receives the event-timed mean.
int b200_bench_mul_mat_q8(int type, int64_t n, int64_t k, int64_t m, const void *const *dev_w, int n_w, const void *dev_act, int act_kind,
                          float *dev_dst, int reps, float *us_per_launch) {
    B200_REQUIRE(dev_w && n_w > 0 && reps > 0 && us_per_launch, "bench_mul_mat_q8: bad arguments");
    cudaStream_t s = nullptr;
    B200_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    int rc = B200_STATUS_SUCCESS;
    for (int i = 0; i < n_w && rc == B200_STATUS_SUCCESS; i++)   // eager first: attributes, error word, scratch
        rc = b200_mul_mat_q8(type, n, k, m, dev_w[i], dev_act, act_kind, dev_dst, n, B200_ROUTE_AUTO, s);
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t e = cudaSuccess;
    if (rc == B200_STATUS_SUCCESS) e = cudaStreamSynchronize(s);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) {
        for (int i = 0; i < reps && rc == B200_STATUS_SUCCESS; i++)
            rc = b200_mul_mat_q8(type, n, k, m, dev_w[i % n_w], dev_act, act_kind, dev_dst, n, B200_ROUTE_AUTO, s);
        e = cudaStreamEndCapture(s, &graph);
    }
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventCreate(&e0);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventCreate(&e1);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaGraphLaunch(exec, s);   // warm
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventRecord(e0, s);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaGraphLaunch(exec, s);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventRecord(e1, s);
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventSynchronize(e1);
    float ms = 0.0f;
    if (rc == B200_STATUS_SUCCESS && e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaStreamDestroy(s);
    if (rc != B200_STATUS_SUCCESS) return rc;
    B200_CUDA(e);
    *us_per_launch = ms * 1e3f / (float)reps;
    return B200_STATUS_SUCCESS;
}

int b200_mul_mat_q8_multi(int type, int64_t k, int count, const int64_t *n, const void *const *dev_w, const void *dev_act, int act_kind,
                          float *const *dev_dst, void *stream) {
    B200_REQUIRE(type == B200_TYPE_Q4_K, "mul_mat_q8_multi: weight type %d is not supported (Q4_K only)", type);
    B200_REQUIRE(count >= 1 && count <= 3 && n && dev_w && dev_dst && dev_act, "mul_mat_q8_multi: bad arguments");
    for (int i = 0; i < count; i++) {
        int rc = check_mul_mat_args(type, n[i], k, 1);
        if (rc != B200_STATUS_SUCCESS) return rc;
        B200_REQUIRE(pick_route(type, n[i], 1) == B200_ROUTE_REPACK, "mul_mat_q8_multi: matrix %d (%lld rows) does not take the 8x8 gemv route",
                     i, (long long)n[i]);
    }
    B200_REQUIRE(act_kind == act_kind_for(type, B200_ROUTE_REPACK, 1), "mul_mat_q8_multi: activation kind %d does not fit type %d", act_kind, type);
    ActView a = act_carve(const_cast<void *>(dev_act), 1, k).view();
    return launch_gemv_q4_K_multi(count, n, (const uint8_t *const *)dev_w, dev_dst, k, a, (cudaStream_t)stream);
}

int b200_mul_mat_q8_rows_multi(int type, int64_t k, int64_t m, int count, const int64_t *n, const void *const *dev_w, const void *dev_act, int act_kind,
                               float *const *dev_dst, const int64_t *lddst, void *stream) {
    B200_REQUIRE(count >= 1 && count <= 3 && n && dev_w && dev_dst && lddst && dev_act, "mul_mat_q8_rows_multi: bad arguments");
    if (m == 0) return B200_STATUS_SUCCESS;
    int route = -1;
    for (int i = 0; i < count; i++) {
        int rc = check_mul_mat_args(type, n[i], k, m);
        if (rc != B200_STATUS_SUCCESS) return rc;
        B200_REQUIRE(dev_w[i] && dev_dst[i] && lddst[i] >= n[i], "mul_mat_q8_rows_multi: matrix %d: null pointer or dst row stride smaller than n", i);
        const int r = pick_route(type, n[i], m);
        B200_REQUIRE(route < 0 || r == route, "mul_mat_q8_rows_multi: matrix %d (%lld rows) takes another route than matrix 0", i, (long long)n[i]);
        route = r;
    }
    B200_REQUIRE(act_kind == act_kind_for(type, route, m), "mul_mat_q8_rows_multi: activation kind %d does not fit type %d", act_kind, type);
    ActBuf a = act_carve(const_cast<void *>(dev_act), m, k);
    return launch_gemv_rows_multi(type, route, count, n, k, m, (const uint8_t *const *)dev_w, a.view(), dev_dst, lddst, (cudaStream_t)stream);
}

int b200_mul_mat_row_fused(int type, int64_t k, int count, const int64_t *n, const void *const *dev_w, float *const *dev_dst,
                           const struct b200_act_prologue *pro, const float *dev_addend, float *dev_sum, void *stream) {
    B200_REQUIRE(type == B200_TYPE_Q4_K, "mul_mat_row_fused: weight type %d is not supported (Q4_K only)", type);
    B200_REQUIRE(count >= 1 && count <= 3 && n && dev_w && dev_dst && pro, "mul_mat_row_fused: bad arguments");
    B200_REQUIRE(pro->mode >= B200_ACT_PRO_PLAIN && pro->mode <= B200_ACT_PRO_SILU && pro->x, "mul_mat_row_fused: bad prologue");
    B200_REQUIRE(pro->mode == B200_ACT_PRO_PLAIN || (pro->w && pro->y_mul), "mul_mat_row_fused: the prologue needs its second operand and its result tensor");
    B200_REQUIRE((dev_addend == nullptr) == (dev_sum == nullptr) && (dev_sum == nullptr || count == 1), "mul_mat_row_fused: the residual add goes with a single matrix");
    const auto al16 = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
    B200_REQUIRE(al16(pro->x) && al16(pro->w) && al16(pro->y) && al16(pro->y_mul), "mul_mat_row_fused: prologue rows must be 16-byte aligned");
    for (int i = 0; i < count; i++) {
        int rc = check_mul_mat_args(type, n[i], k, 1);
        if (rc != B200_STATUS_SUCCESS) return rc;
        B200_REQUIRE(pick_route(type, n[i], 1) == B200_ROUTE_REPACK, "mul_mat_row_fused: matrix %d (%lld rows) does not take the 8x8 gemv route", i,
                     (long long)n[i]);
    }
    ActPrologue p;
    p.mode = pro->mode;
    p.x = pro->x;
    p.w = pro->w;
    p.eps = pro->eps;
    p.wide_end = pro->wide ? (int)(k & ~(int64_t)15) : 0;
    p.y = pro->y;
    p.y_mul = pro->y_mul;
    if (pro->dev_act_out) {
        B200_REQUIRE(((uintptr_t)pro->dev_act_out & 255) == 0, "mul_mat_row_fused: the activation scratch must be 256-byte aligned");
        p.act_out = act_carve(pro->dev_act_out, 1, k);
    }
    ActView a;
    a.qs = nullptr; a.d = nullptr; a.bsums = nullptr; a.dh = nullptr; a.k = k;
    a.addend = dev_addend;
    a.sum = dev_sum;
    return launch_gemv_q4_K_row_fused(count, n, (const uint8_t *const *)dev_w, dev_dst, k, a, p, (cudaStream_t)stream);
}

int b200_mul_mat_q8_add(int type, int64_t n, int64_t k, const void *dev_w, const void *dev_act, int act_kind, float *dev_dst,
                        const float *dev_addend, float *dev_sum, int route, void *stream) {
    int rc = check_mul_mat_args(type, n, k, 1);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (n == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_w && dev_act && dev_dst && dev_addend && dev_sum, "mul_mat_q8_add: null pointer");
    if (route == B200_ROUTE_AUTO) route = pick_route(type, n, 1);
    B200_REQUIRE(act_kind == act_kind_for(type, route, 1), "mul_mat_q8_add: activation kind %d does not fit type %d", act_kind, type);
    ActView a = act_carve(const_cast<void *>(dev_act), 1, k).view();
    a.addend = dev_addend;
    a.sum = dev_sum;
    return launch_gemv(type, route, n, k, 1, (const uint8_t *)dev_w, a, dev_dst, n, (cudaStream_t)stream);
}

int b200_mul_mat_q8_rows_add_fusable(int type, int64_t n, int64_t m) {
    if (!is_quant_type(type) || n <= 0 || m <= 0) return 0;
    return gemv_rows_add_fusable(type, pick_route(type, n, m), m) ? 1 : 0;
}

int b200_mul_mat_q8_rows_add(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const void *dev_act, int act_kind, float *dev_dst, int64_t lddst,
                             const float *dev_addend, int64_t ld_addend, float *dev_sum, int64_t ld_sum, void *stream) {
    int rc = check_mul_mat_args(type, n, k, m);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_w && dev_act && dev_dst && dev_addend && dev_sum, "mul_mat_q8_rows_add: null pointer");
    B200_REQUIRE(lddst >= n && ld_addend >= n && ld_sum >= n, "mul_mat_q8_rows_add: row strides smaller than the rows");
    const int route = pick_route(type, n, m);
    B200_REQUIRE(gemv_rows_add_fusable(type, route, m), "mul_mat_q8_rows_add: type %d with %lld activation rows does not take a few-rows kernel", type, (long long)m);
    B200_REQUIRE(act_kind == act_kind_for(type, route, m), "mul_mat_q8_rows_add: activation kind %d does not fit type %d", act_kind, type);
    ActView a = act_carve(const_cast<void *>(dev_act), m, k).view();
    a.addend = dev_addend;
    a.sum = dev_sum;
    a.ld_addend = ld_addend;
    a.ld_sum = ld_sum;
    return launch_gemv(type, route, n, k, m, (const uint8_t *)dev_w, a, dev_dst, lddst, (cudaStream_t)stream);
}

int b200_mul_mat(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const float *dev_x, int64_t ldx,
                 float *dev_dst, int64_t lddst, int route, void *stream) {
    B200_REQUIRE(is_quant_type(type), "mul_mat: weight type %d is not supported", type);
    B200_REQUIRE(n >= 0 && m >= 0 && k > 0, "mul_mat: bad shape n=%lld k=%lld m=%lld", (long long)n, (long long)k,
                 (long long)m);
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_w && dev_x && dev_dst, "mul_mat: null pointer");
    B200_REQUIRE(ldx >= k && lddst >= n, "mul_mat: row strides smaller than the rows");
    if (route == B200_ROUTE_AUTO) route = pick_route(type, n, m);
    cudaStream_t s = (cudaStream_t)stream;
    void *scratch = nullptr;
    int rc = scratch_get(act_scratch_bytes(m, k), &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    ActBuf a = act_carve(scratch, m, k);
    const int kind = act_kind_for(type, route, m);
    rc = launch_quantize_acts(kind, m, k, dev_x, ldx, a, s);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_gemv(type, route, n, k, m, (const uint8_t *)dev_w, a.view(), dev_dst, lddst, s);
}

int b200_mul_mat_host(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const float *host_x,
                      float *host_dst, int route, void *stream) {
    B200_REQUIRE(n >= 0 && m >= 0 && k > 0, "mul_mat_host: bad shape");
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t xb = (size_t)m * k * 4, ob = (size_t)m * n * 4;
    // the activation scratch sits in front, the f32 staging behind it
    const size_t act_b = act_scratch_bytes(m, k);
    void *scratch = nullptr;
    int rc = scratch_get(act_b + xb + ob + 512, &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    float *dx = (float *)((uint8_t *)scratch + act_b);
    float *dout = (float *)((uint8_t *)dx + (xb + 255) / 256 * 256);
    B200_CUDA(cudaMemcpyAsync(dx, host_x, xb, cudaMemcpyHostToDevice, s));
    rc = b200_mul_mat(type, n, k, m, dev_w, dx, k, dout, n, route, stream);
    if (rc != B200_STATUS_SUCCESS) return rc;
    B200_CUDA(cudaMemcpyAsync(host_dst, dout, ob, cudaMemcpyDeviceToHost, s));
    B200_CUDA(cudaStreamSynchronize(s));
    return B200_STATUS_SUCCESS;
}

int b200_mul_mat_id(int type, int64_t n, int64_t k, int64_t n_expert, int64_t ne11, int64_t n_tok, int64_t n_ids,
                    const void *dev_as, const float *dev_b, const int32_t *dev_ids, float *dev_dst, int route,
                    void *stream) {
    (void)route;  // the route follows from the expert type and shape as in the reference
    B200_REQUIRE(is_quant_type(type), "mul_mat_id: expert type %d is not supported", type);
    B200_REQUIRE(n >= 0 && k > 0 && n_expert > 0 && ne11 > 0 && n_tok >= 0 && n_ids >= 0, "mul_mat_id: bad shape");
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat_id: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || n_tok == 0 || n_ids == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_as && dev_b && dev_ids && dev_dst, "mul_mat_id: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t rows = ne11 * n_tok;   // every b row is quantized once (compute.rs:1952-1985)
    const size_t act_b = act_scratch_bytes(rows, k);
    void *scratch = nullptr;
    const size_t lists_b = mmid_grouped_scratch_bytes(n_expert, n_tok * n_ids);   // covers the per-expert counters of the per-pair path too
    int rc = scratch_get(act_b + lists_b + 256, &scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    ActBuf a = act_carve(scratch, rows, k);
    int *counts = (int *)((uint8_t *)scratch + (act_b + 255) / 256 * 256);
    // rows in passes of 65535 (one launch's grid.y limit)
    for (int64_t r0 = 0; r0 < rows; r0 += 65535) {
        const int64_t nr = rows - r0 < 65535 ? rows - r0 : 65535;
        ActBuf ar = a;
        ar.qs += r0 * k;
        ar.d += r0 * (k / 256);
        ar.bsums += r0 * (k / 16);
        ar.dh += r0 * (k / 32);
        rc = launch_quantize_acts(is_k_quant(type) ? B200_ACT_Q8_K : B200_ACT_Q8_0, nr, k, dev_b + r0 * k, k, ar, s);
        if (rc != B200_STATUS_SUCCESS) return rc;
    }
    return launch_mul_mat_id(type, n, k, n_expert, ne11, n_tok, n_ids, (const uint8_t *)dev_as, a.view(), dev_ids, dev_dst,
                             counts, s);
}



}  // extern "C"
