// FLASH_ATTN_EXT, fast mode, prompt batches (64 and more query rows): tensor-core attention.
//
// The faithful prompt kernel (flash_attn_tiled.cu) reproduces the CPU path's arithmetic position by position on the
// CUDA cores: right to the bit, and two orders of magnitude below what the GPU can do with the same function
//   softmax(q k^T * scale + mask) v        (crates/ggml/src/flash_attn.rs:482-736)
// This is the mode for hosts that accept the tolerance asked of F16-KV attention (1e-3):
//   * a CTA takes 64 rows of one KV head, a row being (token, query head of the KV head's group) with the heads of a
//     token adjacent: the n_head / n_head_kv heads share every K / V tile the CTA stages and every mask row it reads;
//   * q is rounded to f16 as the CPU rounds it (flash_attn.rs:433) and kept in registers as the A fragments of
//     mma.sync m16n8k16; K and V tiles of 64 positions come into shared memory with 16-byte cp.async copies, double
//     buffered, together with the tile's mask rows; K is read with ldmatrix (its rows are the B columns of q k^T), V with
//     ldmatrix.trans (its rows are the B rows of p v);
//   * scores and p v accumulate in f32, softmax runs online per row with exp2, p is rounded to f16 for the second
//     product straight from the accumulator registers (the accumulator layout of one product is the A layout of the next);
//   * a tile in which none of the CTA's rows sees anything (the causal future) costs its copies and one vote.
// Not handled here (the caller falls back to the faithful kernels): sinks, ALiBi, softcap, dk != dv.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int FP_BM = 64;            // rows per CTA (4 warps x 16)
constexpr int FP_BN = 64;            // positions per tile
constexpr int FP_WARPS = 4;
constexpr int FP_MAX_TOK = FP_BM;    // most tokens a row block can span (group 1)
constexpr float FP_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
// d += a (16 x 16, row) * b (16 x 8, col), f16 in, f32 accumulate
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *(const uint32_t *)&h;
}

template <int D>
__global__ void __launch_bounds__(FP_WARPS * 32)
fa_prefill_kernel(b200_flash_attn_args a, int group, float scale_log2) {
    constexpr int PITCH = D * 2 + 16;          // bytes per staged K / V row: the padding keeps ldmatrix rows on different banks
    constexpr int MPITCH = FP_BN * 2 + 16;     // bytes per staged mask row
    constexpr int KS = D / 16;                 // k steps of q k^T
    constexpr int NB = FP_BN / 8;              // score blocks of 8 positions
    constexpr int DB = D / 8;                  // output blocks of 8 value elements
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char *ks = smem;                                   // [2][FP_BN][PITCH]
    unsigned char *vs = ks + 2 * FP_BN * PITCH;                 // [2][FP_BN][PITCH]
    unsigned char *ms = vs + 2 * FP_BN * PITCH;                 // [2][FP_MAX_TOK][MPITCH]

    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = blockIdx.y;
    const int64_t rows_total = a.n_tok * group;
    const int64_t row0 = (int64_t)blockIdx.x * FP_BM;
    const int64_t tok0 = row0 / group;
    int64_t tok_last = (row0 + FP_BM - 1) / group;
    if (tok_last >= a.n_tok) tok_last = a.n_tok - 1;
    const int n_tok_blk = (int)(tok_last - tok0 + 1);           // mask rows this CTA reads
    const int64_t n_tiles = (a.n_kv + FP_BN - 1) / FP_BN;
    const unsigned char *kbase = (const unsigned char *)a.k + (int64_t)hk * a.k_nb2;
    const unsigned char *vbase = (const unsigned char *)a.v + (int64_t)hk * a.v_nb2;

    auto stage = [&](int64_t tile, int buf) {
        constexpr int PIECES = D / 8;   // 16-byte pieces per row
        for (int i = tid; i < FP_BN * PIECES; i += FP_WARPS * 32) {
            const int p = i / PIECES, c = i % PIECES;
            int64_t pos = tile * FP_BN + p;
            if (pos >= a.n_kv) pos = a.n_kv - 1;   // a ragged last tile re-reads the last row; its scores are masked below
            cp16(ks + ((size_t)buf * FP_BN + p) * PITCH + c * 16, kbase + pos * a.k_nb1 + c * 16);
            cp16(vs + ((size_t)buf * FP_BN + p) * PITCH + c * 16, vbase + pos * a.v_nb1 + c * 16);
        }
        if (a.mask) {
            // FP_BN halves = 8 pieces per token row; a ragged tile or an unaligned row start takes 2-byte loads instead
            const bool whole = (tile + 1) * FP_BN <= a.n_kv && (a.mask_nb1 % 16) == 0 && ((uintptr_t)a.mask % 16) == 0;
            for (int i = tid; i < n_tok_blk * 8; i += FP_WARPS * 32) {
                const int t = i / 8, c = i % 8;
                const unsigned char *src = (const unsigned char *)a.mask + (tok0 + t) * a.mask_nb1 + (tile * FP_BN) * 2 + c * 16;
                unsigned char *dst = ms + ((size_t)buf * FP_MAX_TOK + t) * MPITCH + c * 16;
                if (whole) {
                    cp16(dst, src);
                } else {
                    for (int e = 0; e < 8; e++) {
                        const int64_t pos = tile * FP_BN + c * 8 + e;
                        ((uint16_t *)dst)[e] = pos < a.n_kv ? ((const uint16_t *)src)[e] : (uint16_t)0xFC00;   // -inf past the end
                    }
                }
            }
        }
        cp_commit();
    };

    pdl_wait();   // q, the cache rows of this step and the mask come from earlier kernels / copies
    // this thread's rows: r_lo = lane / 4 and r_lo + 8 of the warp's 16
    const int64_t row_a = row0 + warp * 16 + (lane >> 2), row_b = row_a + 8;
    const bool live_a = row_a < rows_total, live_b = row_b < rows_total;
    const int64_t tok_a = live_a ? row_a / group : tok0, tok_b = live_b ? row_b / group : tok0;
    // q as A fragments: for k step s, registers {row a cols 16 s + 2 (lane % 4) .., row b same, row a cols + 8, row b cols + 8}
    uint32_t qf[KS][4];
    {
        const int ha = hk * group + (int)(live_a ? row_a % group : 0), hb = hk * group + (int)(live_b ? row_b % group : 0);
        const float *qa = (const float *)((const unsigned char *)a.q + tok_a * a.q_nb1 + (int64_t)ha * a.q_nb2);
        const float *qb = (const float *)((const unsigned char *)a.q + tok_b * a.q_nb1 + (int64_t)hb * a.q_nb2);
        const int c0 = 2 * (lane & 3);
#pragma unroll
        for (int s = 0; s < KS; s++) {
            const float2 a0 = live_a ? *(const float2 *)(qa + 16 * s + c0) : make_float2(0.f, 0.f);
            const float2 a1 = live_a ? *(const float2 *)(qa + 16 * s + c0 + 8) : make_float2(0.f, 0.f);
            const float2 b0 = live_b ? *(const float2 *)(qb + 16 * s + c0) : make_float2(0.f, 0.f);
            const float2 b1 = live_b ? *(const float2 *)(qb + 16 * s + c0 + 8) : make_float2(0.f, 0.f);
            qf[s][0] = pack_h2(a0.x, a0.y);
            qf[s][1] = pack_h2(b0.x, b0.y);
            qf[s][2] = pack_h2(a1.x, a1.y);
            qf[s][3] = pack_h2(b1.x, b1.y);
        }
    }
    float o[DB][4];
#pragma unroll
    for (int j = 0; j < DB; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;   // running maximum (log2 units) and sum per row (this thread's share)

    // ldmatrix addressing.  K (non-transposed, matrices = 8 positions x 8 halves): lanes 0-7 / 8-15 / 16-23 / 24-31 give the
    // rows of (positions n, halves 0-7), (n, 8-15), (n + 8, 0-7), (n + 8, 8-15): registers b0, b1 of score block n and of n + 8.
    const int k_row = (lane & 7) + ((lane >> 4) << 3), k_col = ((lane >> 3) & 1) * 16;
    // V (transposed, matrices = 8 positions x 8 value halves): lanes give the rows of (positions p, elements e 0-7),
    // (p + 8, e), (p, e + 8), (p + 8, e + 8): registers b0, b1 of output block e and of e + 8.
    const int v_row = (lane & 7) + (((lane >> 3) & 1) << 3), v_col = (lane >> 4) * 16;

    stage(0, 0);
    for (int64_t tile = 0; tile < n_tiles; tile++) {
        const int buf = (int)(tile & 1);
        cp_wait<0>();
        __syncthreads();   // tile `tile` has landed for everyone, and everyone is done with the other buffer
        if (tile + 1 < n_tiles) stage(tile + 1, buf ^ 1);
        // does any row of the CTA see anything in this tile?
        const unsigned char *mt = ms + (size_t)buf * FP_MAX_TOK * MPITCH;
        int any = 0;
        if (a.mask) {
            for (int i = tid; i < n_tok_blk * (FP_BN / 2); i += FP_WARPS * 32) {
                const int t = i / (FP_BN / 2), c = i % (FP_BN / 2);
                const uint32_t two = *(const uint32_t *)(mt + (size_t)t * MPITCH + c * 4);
                any |= ((two & 0xffffu) != 0xFC00u) | ((two >> 16) != 0xFC00u);
            }
        } else {
            any = 1;
        }
        if (!__syncthreads_or(any)) continue;

        // scores of the warp's 16 rows against the tile's 64 positions
        float s[NB][4];
#pragma unroll
        for (int n = 0; n < NB; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
        const unsigned char *kt = ks + (size_t)buf * FP_BN * PITCH;
#pragma unroll
        for (int st = 0; st < KS; st++) {
#pragma unroll
            for (int n = 0; n < NB; n += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, kt + (size_t)(n * 8 + k_row) * PITCH + st * 32 + k_col);
                mma16816(s[n], qf[st], b0, b1);
                mma16816(s[n + 1], qf[st], b2, b3);
            }
        }
        // scale, mask, row maxima
        const unsigned char *ma = mt + (size_t)(tok_a - tok0) * MPITCH, *mb = mt + (size_t)(tok_b - tok0) * MPITCH;
        float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
        for (int n = 0; n < NB; n++) {
            const int c = n * 8 + 2 * (lane & 3);
            float ma0 = 0.0f, ma1 = 0.0f, mb0 = 0.0f, mb1 = 0.0f;
            if (a.mask) {
                const __half2 ha = *(const __half2 *)(ma + c * 2), hb = *(const __half2 *)(mb + c * 2);
                ma0 = __low2float(ha); ma1 = __high2float(ha); mb0 = __low2float(hb); mb1 = __high2float(hb);
            } else if (tile * FP_BN + c + 1 >= a.n_kv) {
                if (tile * FP_BN + c >= a.n_kv) ma0 = mb0 = -INFINITY;
                ma1 = mb1 = -INFINITY;
            }
            s[n][0] = live_a ? fmaf(s[n][0], scale_log2, ma0 * FP_LOG2E) : -INFINITY;
            s[n][1] = live_a ? fmaf(s[n][1], scale_log2, ma1 * FP_LOG2E) : -INFINITY;
            s[n][2] = live_b ? fmaf(s[n][2], scale_log2, mb0 * FP_LOG2E) : -INFINITY;
            s[n][3] = live_b ? fmaf(s[n][3], scale_log2, mb1 * FP_LOG2E) : -INFINITY;
            mx_a = fmaxf(mx_a, fmaxf(s[n][0], s[n][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[n][2], s[n][3]));
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
        // a row that has seen nothing yet keeps a zero accumulator; exp2(-inf - -inf) must not be formed
        const float al_a = m_a == -INFINITY ? 0.0f : exp2f(m_a - mn_a), al_b = m_b == -INFINITY ? 0.0f : exp2f(m_b - mn_b);
        const float sub_a = mn_a == -INFINITY ? 0.0f : mn_a, sub_b = mn_b == -INFINITY ? 0.0f : mn_b;
        m_a = mn_a; m_b = mn_b;
        float ps_a = 0.0f, ps_b = 0.0f;
        uint32_t pf[NB / 2][4];   // p as A fragments of the second product: k step j = score blocks 2 j and 2 j + 1
#pragma unroll
        for (int n = 0; n < NB; n++) {
            const float p0 = exp2f(s[n][0] - sub_a), p1 = exp2f(s[n][1] - sub_a), p2 = exp2f(s[n][2] - sub_b), p3 = exp2f(s[n][3] - sub_b);
            const __half2 ha = __floats2half2_rn(p0, p1), hb = __floats2half2_rn(p2, p3);
            // the row sum takes the weights as the second product will see them (rounded to f16): numerator and
            // denominator then carry the same rounding, and what is common to a row's weights cancels
            const float2 fa = __half22float2(ha), fb = __half22float2(hb);
            ps_a += fa.x + fa.y;
            ps_b += fb.x + fb.y;
            pf[n >> 1][(n & 1) * 2 + 0] = *(const uint32_t *)&ha;
            pf[n >> 1][(n & 1) * 2 + 1] = *(const uint32_t *)&hb;
        }
        l_a = fmaf(l_a, al_a, ps_a);
        l_b = fmaf(l_b, al_b, ps_b);
#pragma unroll
        for (int j = 0; j < DB; j++) {
            o[j][0] *= al_a; o[j][1] *= al_a; o[j][2] *= al_b; o[j][3] *= al_b;
        }
        const unsigned char *vt = vs + (size_t)buf * FP_BN * PITCH;
#pragma unroll
        for (int j = 0; j < FP_BN / 16; j++) {
#pragma unroll
            for (int e = 0; e < DB; e += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, vt + (size_t)(j * 16 + v_row) * PITCH + e * 16 + v_col);
                mma16816(o[e], pf[j], b0, b1);
                mma16816(o[e + 1], pf[j], b2, b3);
            }
        }
    }
    cp_wait<0>();
    // the four threads of a row hold parts of its sum
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;   // a row that sees nothing gives zeros, as on the CPU
    const int c0 = 2 * (lane & 3);
    if (live_a) {
        float *dst = a.dst + (tok_a * a.n_head + hk * group + row_a % group) * D;
#pragma unroll
        for (int j = 0; j < DB; j++) *(float2 *)(dst + j * 8 + c0) = make_float2(o[j][0] * inv_a, o[j][1] * inv_a);
    }
    if (live_b) {
        float *dst = a.dst + (tok_b * a.n_head + hk * group + row_b % group) * D;
#pragma unroll
        for (int j = 0; j < DB; j++) *(float2 *)(dst + j * 8 + c0) = make_float2(o[j][2] * inv_b, o[j][3] * inv_b);
    }
}

}  // namespace

// true: the fast prompt kernel took the call (*rc is its status); false: not a shape it handles
bool flash_attn_fast_prefill(const b200_flash_attn_args *a, cudaStream_t s, int *rc) {
    *rc = B200_STATUS_SUCCESS;
    if (a->sinks || a->max_bias != 0.0f || a->logit_softcap != 0.0f || a->dk != a->dv || (a->dk != 64 && a->dk != 128) || a->n_kv == 0 || a->n_tok == 0)
        return false;
    if (a->q_nb1 % 8 || a->q_nb2 % 8 || ((uintptr_t)a->q & 7) || ((uintptr_t)a->dst & 7) || a->n_head % a->n_head_kv) return false;
    if (a->k_nb1 % 16 || a->v_nb1 % 16 || a->k_nb2 % 16 || a->v_nb2 % 16 || ((uintptr_t)a->k & 15) || ((uintptr_t)a->v & 15)) return false;
    if (a->mask && (a->mask_nb1 % 2 || ((uintptr_t)a->mask & 1))) return false;
    const int group = (int)(a->n_head / a->n_head_kv);
    const int64_t rows = a->n_tok * group;
    const int64_t row_blocks = (rows + FP_BM - 1) / FP_BM;
    if (row_blocks > 0x7fffffffLL || a->n_head_kv > 65535) return false;
    const int D = (int)a->dk;
    const size_t smem = (size_t)4 * FP_BN * (D * 2 + 16) + (size_t)2 * FP_MAX_TOK * (FP_BN * 2 + 16);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        *rc = cuda_fail(cudaGetLastError(), "flash_attn prefill: device query", __FILE__, __LINE__);
        return true;
    }
    static bool attr_done[64][2] = {};
    if (!attr_done[dev][D == 128]) {
        cudaError_t e = D == 128 ? cudaFuncSetAttribute(fa_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                 : cudaFuncSetAttribute(fa_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { *rc = cuda_fail(e, "cudaFuncSetAttribute", __FILE__, __LINE__); return true; }
        attr_done[dev][D == 128] = true;
    }
    const dim3 grid((unsigned)row_blocks, (unsigned)a->n_head_kv);
    const float scale_log2 = a->scale * FP_LOG2E;
    if (D == 128) *rc = launch_pdl(fa_prefill_kernel<128>, grid, dim3(FP_WARPS * 32), smem, s, *a, group, scale_log2);
    else *rc = launch_pdl(fa_prefill_kernel<64>, grid, dim3(FP_WARPS * 32), smem, s, *a, group, scale_log2);
    return true;
}

}  // namespace b200
