// Q4_K decode mat-mul, streaming version: persistent CTAs, an asynchronous
// bulk-copy ring in shared memory, programmatic dependent launch.
//
// Same arithmetic as gemv_q4_K_kernel<1, 0> (bit-identical to the CPU's 8x8
// gemv, crates/ggml/src/repack.rs:1638-1688); what changes is how the bytes move:
//   * one CTA per SM walks row tiles blockIdx.x, blockIdx.x + gridDim.x, ...;
//   * one producer thread issues one cp.async.bulk per ring stage (36864
//     contiguous bytes = eight consecutive (tile, 256-element group) chunks of
//     the tile layout; measured on B200 a bulk copy costs about 350 ns per SM
//     whatever its size or the number in flight, so 4608-byte copies cap an SM
//     at 13 GB/s and 18 KB ones only just reach its share of the HBM rate),
//     each completing on the stage's
//     mbarrier, so several stages per SM are in flight with no registers tied
//     up and the memory pipe does not drain between tiles;
//   * consumer warps (lane = row) read their chunk from shared memory, do the
//     dp4a block dots against the activations (staged once per CTA), leave the
//     int32 partials in a double-buffered exchange array, and release the stage;
//   * the warp that completes a tile's last group runs the tile's f32 chains in
//     K order and stores the 32 outputs;
//   * the kernel is launched with the programmatic-stream-serialization
//     attribute: its weight prefetch starts while the previous kernel in the
//     stream is still finishing; activations are read only after
//     griddepcontrol.wait.
// Every wait is bounded: on expiry the thread records an error code in
// *err_flag and the CTA winds down without touching the output.
#include <cstdlib>

#include "common.cuh"

namespace b200 {

namespace {

constexpr int CHUNK = 4608;
constexpr int STAGE_GROUPS = 8;                       // groups (chunks) per bulk copy
constexpr int STAGE_BYTES = STAGE_GROUPS * CHUNK;     // 36864
constexpr int MAX_STAGES = 16;
constexpr int MAX_XB = 4;                             // exchange buffers (tiles in flight)
// Consumer warps form CW / STAGE_GROUPS sets of STAGE_GROUPS warps.  Units (stages' worth of groups) go
// to the sets round-robin and the ring depth is a multiple of the set count, so a ring stage is always
// consumed by the same warps: every waiter sees every phase of its barriers in order, which is what
// makes the parity waits unambiguous (a thread that waited two phases ahead would fall through).
constexpr unsigned SPIN_LIMIT = 1u << 20;             // polls with a short sleep between them: about a second in all

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait for the phase with the given parity; false on expiry
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, unsigned limit = SPIN_LIMIT) {
    const uint32_t a = smem_u32(bar);
    for (unsigned i = 0; i < limit; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        if (i > 4) __nanosleep(64);   // keep the pollers off the shared-memory pipe the workers need
    }
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

struct StreamSmem {
    // dynamic layout: ring[stages][STAGE_BYTES] | acts.qs[k] | bp[nb][8] | dx[nb] | xch[xb][nb][32] int4 | barriers
    uint8_t *ring;
    int8_t *aq;
    int *bp;
    float *dx;
    int *xch;        // [xb][3 planes: iacc, imin, d|dmin][nb][32]
    uint64_t *full, *empty;
    int *tile_cnt;   // [MAX_XB]
    int *abort_flag;
};

__host__ __device__ inline size_t stream_fixed_bytes(int nb, int xb) {
    return (size_t)nb * 256 + (size_t)nb * 32 + ((size_t)nb * 4 + 15) / 16 * 16 + (size_t)xb * nb * 32 * 12 +
           2 * MAX_STAGES * 8 + 64;
}

__device__ __forceinline__ StreamSmem carve(unsigned char *base, int stages, int nb, int xb) {
    StreamSmem s;
    s.ring = base;
    base += (size_t)stages * STAGE_BYTES;
    s.aq = (int8_t *)base;
    base += (size_t)nb * 256;
    s.bp = (int *)base;
    base += (size_t)nb * 8 * 4;
    s.dx = (float *)base;
    base += (((size_t)nb * 4) + 15) / 16 * 16;
    s.xch = (int *)base;
    base += (size_t)xb * nb * 32 * 12;
    s.full = (uint64_t *)base;
    base += MAX_STAGES * 8;
    s.empty = (uint64_t *)base;
    base += MAX_STAGES * 8;
    s.tile_cnt = (int *)base;
    s.abort_flag = s.tile_cnt + MAX_XB;
    return s;
}

template <int CONSUMER_WARPS>
__global__ void __launch_bounds__((CONSUMER_WARPS + 1) * 32, 1)
gemv_q4_K_stream_kernel(const uint8_t *__restrict__ tiles, ActView acts, float *__restrict__ dst, int64_t n, int nb,
                        int n_tiles, int stages, int xb, int *err_flag, unsigned spin_limit, int skip_unit) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    StreamSmem sm = carve(smem_raw, stages, nb, xb);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int spt = (nb + STAGE_GROUPS - 1) / STAGE_GROUPS;   // stages (units) per tile
    const int my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1 - blockIdx.x) / gridDim.x + 1 : 0;
    const int64_t units = (int64_t)my_tiles * spt;

    if (tid == 0) {
        for (int i = 0; i < stages; i++) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], STAGE_GROUPS);   // one arrival per group slot of the stage
        }
        for (int i = 0; i < MAX_XB; i++) sm.tile_cnt[i] = 0;
        *sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // let the next kernel in the stream begin its own prologue
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // the producer lane's record of what it put in flight: stages used at least once, and the parity of the last
    // phase it started on each (read again in the wind-down)
    unsigned issued_mask = 0, issued_parity = 0;
    if (warp == CONSUMER_WARPS) {
        // ---------------- producer: weights do not depend on the previous kernel in the stream
        if (lane == 0) {
            // (st, ph): ring stage and phase of unit u; (it, sg): its tile and first group.  All counters
            // advance incrementally: no divisions in the loop.
            int st = 0, sg = 0;
            unsigned ph = 0;
            int64_t tile = blockIdx.x;
            for (int64_t u = 0; u < units; u++) {
                if (u >= stages && !mbar_wait(&sm.empty[st], ph ^ 1, spin_limit)) {
                    atomicExch(err_flag, 1);
                    *(volatile int *)sm.abort_flag = 1;
                    break;
                }
                if (*(volatile int *)sm.abort_flag) break;
                const int ng = nb - sg < STAGE_GROUPS ? nb - sg : STAGE_GROUPS;
                if (u != skip_unit) {   // skip_unit >= 0 only in the wait-expiry test: that stage is never filled
                    mbar_expect_tx(&sm.full[st], (unsigned)ng * CHUNK);
                    bulk_load(sm.ring + (size_t)st * STAGE_BYTES, tiles + (tile * nb + sg) * (int64_t)CHUNK, (unsigned)ng * CHUNK,
                              &sm.full[st]);
                    issued_mask |= 1u << st;
                    issued_parity = (issued_parity & ~(1u << st)) | (ph << st);
                }
                if (++st == stages) { st = 0; ph ^= 1; }
                sg += STAGE_GROUPS;
                if (sg >= nb) { sg = 0; tile += gridDim.x; }
            }
        }
    } else {
        // ---------------- consumers ----------------
        // the activations come from the previous kernel in the stream
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int ctid = tid;   // 0 .. CONSUMER_WARPS*32 - 1
        for (int i = ctid; i < nb * 16; i += CONSUMER_WARPS * 32)
            ((uint4 *)sm.aq)[i] = ((const uint4 *)acts.qs)[i];
        for (int i = ctid; i < nb * 8; i += CONSUMER_WARPS * 32) {
            const short2 s2 = ((const short2 *)acts.bsums)[i];
            sm.bp[i] = (int)s2.x + (int)s2.y;
        }
        for (int i = ctid; i < nb; i += CONSUMER_WARPS * 32) sm.dx[i] = acts.d[i];
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");

        constexpr int NSETS = CONSUMER_WARPS / STAGE_GROUPS;
        const int set = warp / STAGE_GROUPS, wj = warp % STAGE_GROUPS;
        // incremental counters of the set's current unit: ring stage / phase, tile ordinal, exchange
        // buffer, first group of the unit within its tile
        int st = set % stages, sg = 0, xi = 0;
        unsigned ph = 0;
        int64_t tile = blockIdx.x;
        for (int a = 0; a < set; a++) {   // advance to unit `set`
            sg += STAGE_GROUPS;
            if (sg >= nb) { sg = 0; tile += gridDim.x; if (++xi == xb) xi = 0; }
        }
        for (int64_t u = set; u < units; u += NSETS) {
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&sm.full[st], ph, spin_limit);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok || *(volatile int *)sm.abort_flag) {
                if (lane == 0 && !ok) {
                    atomicExch(err_flag, 2);
                    *(volatile int *)sm.abort_flag = 1;
                }
                break;
            }
            const int b = sg + wj;
            if (b < nb) {
                const uint8_t *chunk = sm.ring + (size_t)st * STAGE_BYTES + (size_t)wj * CHUNK;
                const uint4 h = *(const uint4 *)(chunk + lane * 16);
                uint4 q[8];
#pragma unroll
                for (int c = 0; c < 8; c++) q[c] = *(const uint4 *)(chunk + 512 + c * 512 + lane * 16);
                // 6-bit scales and mins: crates/ggml/src/quants.rs:421-429
                const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
                const uint32_t sc_lo4 = u0 & 0x3f3f3f3fu, mn_lo4 = u1 & 0x3f3f3f3fu;
                const uint32_t sc_hi4 = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
                const uint32_t mn_hi4 = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
                const uint4 *aq = (const uint4 *)(sm.aq + (size_t)b * 256);
                int iacc = 0;
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    int dlo = 0, dhi = 0;
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        const uint4 w = q[2 * g + hh];
                        const uint4 alo = aq[4 * g + hh], ahi = aq[4 * g + 2 + hh];
                        dlo = __dp4a((int)(w.x & 0x0f0f0f0fu), (int)alo.x, dlo);
                        dlo = __dp4a((int)(w.y & 0x0f0f0f0fu), (int)alo.y, dlo);
                        dlo = __dp4a((int)(w.z & 0x0f0f0f0fu), (int)alo.z, dlo);
                        dlo = __dp4a((int)(w.w & 0x0f0f0f0fu), (int)alo.w, dlo);
                        dhi = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), (int)ahi.x, dhi);
                        dhi = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), (int)ahi.y, dhi);
                        dhi = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), (int)ahi.z, dhi);
                        dhi = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), (int)ahi.w, dhi);
                    }
                    const uint32_t s4 = g < 2 ? sc_lo4 : sc_hi4;
                    iacc += dlo * (int)((s4 >> (16 * (g & 1))) & 0xff) + dhi * (int)((s4 >> (16 * (g & 1) + 8)) & 0xff);
                }
                int imin = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint32_t m4 = j < 4 ? mn_lo4 : mn_hi4;
                    imin += (int)((m4 >> (8 * (j & 3))) & 0xff) * sm.bp[b * 8 + j];
                }
                int *xt = sm.xch + (size_t)xi * 3 * nb * 32;
                xt[b * 32 + lane] = iacc;
                xt[(nb + b) * 32 + lane] = imin;
                xt[(2 * nb + b) * 32 + lane] = (int)h.x;
                __syncwarp();
                // the group that completes a tile runs the tile's chains before releasing its stage; with
                // stages <= (xb - 1) * spt that keeps the producers out of an unfinished exchange buffer
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(&sm.tile_cnt[xi], 1) == nb - 1;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    __threadfence_block();
                    float sumf = 0.0f, summin = 0.0f;
#pragma unroll 4
                    for (int bb = 0; bb < nb; bb++) {
                        const int vi = xt[bb * 32 + lane], vm = xt[(nb + bb) * 32 + lane];
                        const uint32_t hd = (uint32_t)xt[(2 * nb + bb) * 32 + lane];
                        const float d = f16_bits_to_f32((uint16_t)(hd & 0xffffu));
                        const float dmin = f16_bits_to_f32((uint16_t)(hd >> 16));
                        const float da = sm.dx[bb];
                        sumf = __fmaf_rn((float)vi, __fmul_rn(d, da), sumf);
                        summin = __fmaf_rn((float)vm, __fmul_rn(dmin, da), summin);
                    }
                    const int64_t row = tile * TILE_ROWS + lane;
                    if (row < n) {
                        const float v = __fsub_rn(sumf, summin);
                        dst[row] = v;
                        if (acts.sum) acts.sum[row] = __fadd_rn(v, acts.addend[row]);
                    }
                    if (lane == 0) sm.tile_cnt[xi] = 0;
                    __syncwarp();
                }
            }
            if (lane == 0) mbar_arrive(&sm.empty[st]);
            // step NSETS units ahead
            st += NSETS;
            if (st >= stages) { st -= stages; ph ^= 1; }
#pragma unroll
            for (int a = 0; a < NSETS; a++) {
                sg += STAGE_GROUPS;
                if (sg >= nb) { sg = 0; tile += gridDim.x; if (++xi == xb) xi = 0; }
            }
        }
    }
    // wind-down: every bulk copy this CTA issued must have landed before shared memory is released.  On the
    // normal path the consumers have waited for each of them; after an abort the producer lane waits (bounded)
    // for the last phase it started on every stage.
    __syncthreads();
    if (*(volatile int *)sm.abort_flag && warp == CONSUMER_WARPS && lane == 0) {
        for (int i = 0; i < stages; i++)
            if (issued_mask & (1u << i)) mbar_wait(&sm.full[i], (issued_parity >> i) & 1u, spin_limit < 4096u ? 4096u : spin_limit);
    }
}

}  // namespace

// Device-side error word of the kernels: a file-scope device variable (every device that loads the module holds
// its own zero-initialized copy), so finding it takes no allocation.  In host code the name is only a handle for
// cudaGetSymbolAddress; g_err_flag[dev] is the address kernels get.
static __device__ int g_err_word_dev;
static int *g_err_flag[64] = {nullptr};
// test hook (b200_debug_stream_wait): a poll limit for the streaming kernel's waits and a ring unit its producer
// leaves unfilled, so that a test can watch a wait run out and the kernel return with an error code
static int g_wait_limit_override = 0;
static int g_skip_unit_override = -1;
void gemv_stream_debug_wait(int spin_limit, int skip_unit) {
    g_wait_limit_override = spin_limit > 0 ? spin_limit : 0;
    g_skip_unit_override = skip_unit >= 0 ? skip_unit : -1;
}
// while the hook is armed (a poll limit is set) one-row Q4_K mat-muls take the streaming kernel
bool gemv_stream_forced() { return g_wait_limit_override > 0; }

// the current device's error word; kernels that skip a bad index or give up a wait store a non-zero code there
// and b200_kernel_error() reads and clears it
int device_error_word(int **flag) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "device index %d out of range", dev);
    if (!g_err_flag[dev]) {
        void *p = nullptr;
        B200_CUDA(cudaGetSymbolAddress(&p, g_err_word_dev));
        B200_REQUIRE(p != nullptr, "the device reported no address for the error word");
        g_err_flag[dev] = (int *)p;
    }
    *flag = g_err_flag[dev];
    return B200_STATUS_SUCCESS;
}

// B200_STREAM_VARIANT: 0 (default) = 16 consumer warps, up to 216 KB of shared memory, one CTA per SM;
// 1 = 8 consumer warps and at most 104 KB, so that two CTAs (of this launch, or of this launch and the next one in
// the stream, which starts its weight prefetch early under programmatic dependent launch) share an SM.
int gemv_stream_variant() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200_STREAM_VARIANT");
        v = (e && e[0] == '1') ? 1 : 0;
    }
    return v;
}

template <int CW>
static int launch_stream_variant(int64_t n, int64_t k, const uint8_t *tiles, ActView acts, float *dst, cudaStream_t s, size_t budget,
                                 int ctas_per_sm) {
    const int nb = (int)(k / GROUP_K);
    const int n_tiles = (int)((n + TILE_ROWS - 1) / TILE_ROWS);
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    B200_REQUIRE(dev >= 0 && dev < 64, "gemv stream: device index %d out of range", dev);
    static int sm_count[64] = {0};
    static bool attr_done[64] = {false};
    if (!attr_done[dev]) {
        cudaDeviceProp p;
        B200_CUDA(cudaGetDeviceProperties(&p, dev));
        sm_count[dev] = p.multiProcessorCount;
        B200_CUDA(cudaFuncSetAttribute(gemv_q4_K_stream_kernel<CW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));

        int *flag = nullptr;
        int rc = device_error_word(&flag);
        if (rc != B200_STATUS_SUCCESS) return rc;
        attr_done[dev] = true;
    }
    // exchange buffers and ring stages: the ring may not run more than (xb - 1) tiles ahead of an
    // unfinished tile (see the kernel), and everything has to fit in the shared-memory budget
    constexpr int NSETS = CW / STAGE_GROUPS;
    const int spt = (nb + STAGE_GROUPS - 1) / STAGE_GROUPS;
    int xb = 2, stages = 0;
    for (int cand = MAX_XB; cand >= 2; cand--) {
        const size_t fixed = stream_fixed_bytes(nb, cand);
        if (fixed + (size_t)2 * STAGE_BYTES > budget) continue;
        int st = (int)((budget - fixed) / STAGE_BYTES);
        if (st > (cand - 1) * spt) st = (cand - 1) * spt;
        if (st > MAX_STAGES) st = MAX_STAGES;
        st -= st % NSETS;   // a multiple of the consumer set count
        if (st > stages) { stages = st; xb = cand; }
    }
    B200_REQUIRE(stages >= 2 && stages >= NSETS, "gemv stream: k = %lld leaves no room for the copy ring", (long long)k);
    const size_t smem = stream_fixed_bytes(nb, xb) + (size_t)stages * STAGE_BYTES;
    const int max_ctas = sm_count[dev] * ctas_per_sm;
    const int grid = n_tiles < max_ctas ? n_tiles : max_ctas;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((CW + 1) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    B200_CUDA(cudaLaunchKernelEx(&cfg, gemv_q4_K_stream_kernel<CW>, tiles, acts, dst, n, nb, n_tiles, stages, xb, g_err_flag[dev],
                                 g_wait_limit_override > 0 ? (unsigned)g_wait_limit_override : SPIN_LIMIT, g_skip_unit_override));
    return B200_STATUS_SUCCESS;
}

int launch_gemv_q4_K_stream(int64_t n, int64_t k, const uint8_t *tiles, ActView acts, float *dst, cudaStream_t s) {
    if (gemv_stream_variant() == 1) return launch_stream_variant<8>(n, k, tiles, acts, dst, s, (size_t)104 * 1024, 2);
    return launch_stream_variant<16>(n, k, tiles, acts, dst, s, (size_t)216 * 1024, 1);
}

// 0 = no streaming kernel has given up a wait on this device since the last call
int gemv_stream_error(int *code) {
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    *code = 0;
    if (dev < 0 || dev >= 64 || !g_err_flag[dev]) return B200_STATUS_SUCCESS;
    B200_CUDA(cudaMemcpy(code, g_err_flag[dev], sizeof(int), cudaMemcpyDeviceToHost));
    if (*code) {
        B200_CUDA(cudaMemset(g_err_flag[dev], 0, sizeof(int)));
        return gemm_fast_reset_flags();   // a kernel that gave up may have left partial-tile flags of the fast prompt mat-mul raised
    }
    return B200_STATUS_SUCCESS;
}

}  // namespace b200
