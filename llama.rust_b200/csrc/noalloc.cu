// b200_mul_mat_static_scratch: MUL_MAT for callers that must not allocate.
//
// b200_mul_mat() keeps its quantized activations in a scratch block that the
// library obtains from cudaMalloc on first use and re-allocates when a larger
// one is needed.  Some hosts cannot tolerate that: a real-time decode loop that
// has pinned its memory budget up front, a process running under a memory
// manager that owns every device allocation, or code that runs while the
// allocator is unavailable to it.  For them this entry point does the same
// quantize-then-multiply with the scratch placed in a fixed array that is part
// of the loaded module itself, so no allocation call of any kind happens here:
// the kernels' error word and counters are file-scope device variables too, and
// for the shapes where b200_mul_mat would pick a kernel that needs a further
// scratch block (the two-pass prompt mat-mul with its operand images) this entry
// point runs the one-pass kernel that computes the same bits without it.
//
// Consequences a caller has to know:
//  * the array is B200_STATIC_SCRATCH_BYTES (256 KiB) large and every device
//    that loads the library holds one copy of it until the process exits;
//  * shapes whose quantized activations do not fit are refused with a status
//    and a message, nothing is launched;
//  * the first call on a device looks the array's device address up once
//    (with that device current).  Make that first call before any stream
//    capture is begun on the device;
//  * all calls on a device share the one array and it keeps whatever the last
//    call wrote.  Nothing in it has to start at zero (the quantizer writes
//    every byte the multiply reads), but two calls whose kernels overlap on
//    the GPU (different streams without an ordering between them) race on it.
//    Calls issued into one stream are ordered and safe.
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t STATIC_SCRATCH_BYTES = 256 * 1024;

// Lives in device memory of every device the module is loaded on.  In host
// code this name is only a handle for cudaGetSymbolAddress, never a pointer
// that may be handed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

std::mutex g_mu;
void *g_addr[64] = {nullptr};

int static_scratch_address(void **out) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "static scratch: device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_addr[dev] == nullptr) {
        void *p = nullptr;
        B200_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        B200_REQUIRE(p != nullptr, "static scratch: the device reported no address for the array");
        g_addr[dev] = p;
    }
    *out = g_addr[dev];
    return B200_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

size_t b200_static_scratch_nbytes(void) { return STATIC_SCRATCH_BYTES; }

int b200_mul_mat_static_scratch(int type, int64_t n, int64_t k, int64_t m, const void *dev_w, const float *dev_x,
                                int64_t ldx, float *dev_dst, int64_t lddst, int route, void *stream) {
    using namespace b200;
    B200_REQUIRE(is_quant_type(type), "mul_mat_static_scratch: weight type %d is not supported", type);
    B200_REQUIRE(n >= 0 && m >= 0 && k > 0, "mul_mat_static_scratch: bad shape n=%lld k=%lld m=%lld", (long long)n,
                 (long long)k, (long long)m);
    B200_REQUIRE(k % GROUP_K == 0, "mul_mat_static_scratch: k = %lld must be a multiple of 256", (long long)k);
    if (n == 0 || m == 0) return B200_STATUS_SUCCESS;
    B200_REQUIRE(dev_w && dev_x && dev_dst, "mul_mat_static_scratch: null pointer");
    B200_REQUIRE(ldx >= k && lddst >= n, "mul_mat_static_scratch: row strides smaller than the rows");
    const size_t need = act_scratch_bytes(m, k);
    B200_REQUIRE(need <= STATIC_SCRATCH_BYTES,
                 "mul_mat_static_scratch: %lld x %lld activations need %zu bytes of scratch, the fixed array holds %zu; "
                 "use b200_mul_mat for this shape",
                 (long long)m, (long long)k, need, STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != B200_STATUS_SUCCESS) return rc;
    if (route == B200_ROUTE_AUTO) route = pick_route(type, n, m);
    cudaStream_t s = (cudaStream_t)stream;
    // inside this scope the launchers take only routes that need no further scratch block (the two-pass prompt
    // kernels and the K split are skipped), and any request for library scratch is refused instead of served
    NoScratchScope no_scratch;
    ActBuf a = act_carve(scratch, m, k);
    rc = launch_quantize_acts(act_kind_for(type, route, m), m, k, dev_x, ldx, a, s);
    if (rc != B200_STATUS_SUCCESS) return rc;
    return launch_gemv(type, route, n, k, m, (const uint8_t *)dev_w, a.view(), dev_dst, lddst, s);
}

}  // extern "C"
