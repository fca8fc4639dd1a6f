// AVX2 / AVX-512 VNNI bodies of the two integer cores that carry the CPU baseline of the benchmark: the Q4_K 8x8
// tile core shared by the repack gemv and gemm (crates/ggml/src/repack.rs:1777-, `mod simd_x86_q4k`) and the Q6_K
// row dot (crates/ggml/src/simd_x86.rs:799).  TEST INFRASTRUCTURE / CPU BASELINE, like the rest of oracle/: nothing in
// the product path uses it.
//
// These are this repository's own vector code, not a transcription: the reference's SIMD bodies and its scalar
// specifications are documented as bit-identical to each other, because every integer sub-dot is exact and the
// f32 chain is the same sequence of fused multiply-adds.  The functions here compute the same exact integers as the
// scalar restatement in oracle_matmul.cpp (checked bit for bit by tests/test_oracle_simd.py) and leave the f32
// chains to the callers, unchanged.  The AVX2 forms need only x86-64-v3; the VNNI forms are picked at run time when
// the host has AVX512-VNNI + VL (orc_simd_level reports which).
#include <immintrin.h>
#include <stdint.h>
#include <string.h>

#include "oracle.h"

// Levels: 0 = scalar, 1 = AVX2, 2 = AVX-512 VNNI.  orc_set_simd caps the level (tests walk through all three);
// orc_simd_level is the cap met with what the host has.
static int g_simd_cap = 2;
extern "C" void orc_set_simd(int max_level) { g_simd_cap = max_level < 0 ? 0 : max_level > 2 ? 2 : max_level; }
extern "C" int orc_simd_level() {
    if (g_simd_cap == 0 || !__builtin_cpu_supports("avx2")) return 0;
    const int host = __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl") ? 2 : 1;
    return host < g_simd_cap ? host : g_simd_cap;
}

// Decode one 12-byte group of block_q4_Kx8.scales into the 8 columns' (scale, min):
// crates/ggml/src/repack.rs:1311-1333,1612-1622 (the same unpacking as the scalar restatement)
static inline void q4kx8_scales(const uint8_t *tile, int sb, uint8_t *s, uint8_t *m) {
    const int off = sb < 4 ? 12 * sb : 12 * (sb - 4) + 48;
    uint32_t u[4];
    memcpy(u, tile + 32 + off, 12);
    const uint32_t K1 = 0x3f3f3f3f, K2 = 0x0f0f0f0f, K3 = 0x03030303;
    u[3] = ((u[2] >> 4) & K2) | (((u[1] >> 6) & K3) << 4);
    uint32_t aux = u[1] & K1;
    u[1] = (u[2] & K2) | (((u[0] >> 6) & K3) << 4);
    u[2] = aux;
    u[0] &= K1;
    memcpy(s, &u[0], 8);
    memcpy(m, &u[2], 8);
}

// One (8-row tile, activation super-block): iacc / imin per sub-block pair g for the 8 rows of the tile.
// Inside pair g the tile stores, for each 8-element piece p of the pair's 32-element halves, the 8 rows' 8 bytes one
// after the other (64 bytes): two 256-bit loads cover rows 0-3 and 4-7; low nibbles meet activation elements
// 64 g + 8 p .., high nibbles 64 g + 32 + 8 p ...
__attribute__((target("avx2"))) static void q4kx8_ints_avx2(const uint8_t *tile, const int8_t *q8, const int16_t *bs, int iacc[4][8],
                                                             int imin[4][8]) {
    const __m256i m4 = _mm256_set1_epi8(0x0F), ones = _mm256_set1_epi16(1);
    const __m256i row_order = _mm256_setr_epi32(0, 1, 4, 5, 2, 3, 6, 7);
    for (int g = 0; g < 4; g++) {
        const uint8_t *qs = tile + 128 + 256 * g;
        __m256i lo03 = _mm256_setzero_si256(), lo47 = lo03, hi03 = lo03, hi47 = lo03;
        for (int p = 0; p < 4; p++) {
            const __m256i w03 = _mm256_loadu_si256((const __m256i *)(qs + 64 * p)), w47 = _mm256_loadu_si256((const __m256i *)(qs + 64 * p + 32));
            long long ylo8, yhi8;
            memcpy(&ylo8, q8 + 64 * g + 8 * p, 8);
            memcpy(&yhi8, q8 + 64 * g + 32 + 8 * p, 8);
            const __m256i ylo = _mm256_set1_epi64x(ylo8), yhi = _mm256_set1_epi64x(yhi8);
            // unsigned nibbles x signed quants, pairs added in 16 bits: at most 4 x 2 x 15 x 127 per lane over the 4 pieces
            lo03 = _mm256_add_epi16(lo03, _mm256_maddubs_epi16(_mm256_and_si256(w03, m4), ylo));
            lo47 = _mm256_add_epi16(lo47, _mm256_maddubs_epi16(_mm256_and_si256(w47, m4), ylo));
            hi03 = _mm256_add_epi16(hi03, _mm256_maddubs_epi16(_mm256_and_si256(_mm256_srli_epi16(w03, 4), m4), yhi));
            hi47 = _mm256_add_epi16(hi47, _mm256_maddubs_epi16(_mm256_and_si256(_mm256_srli_epi16(w47, 4), m4), yhi));
        }
        // two dwords per row -> one per row, rows back in order
        const __m256i dlo = _mm256_permutevar8x32_epi32(_mm256_hadd_epi32(_mm256_madd_epi16(lo03, ones), _mm256_madd_epi16(lo47, ones)), row_order);
        const __m256i dhi = _mm256_permutevar8x32_epi32(_mm256_hadd_epi32(_mm256_madd_epi16(hi03, ones), _mm256_madd_epi16(hi47, ones)), row_order);
        uint8_t s_lo[8], m_lo[8], s_hi[8], m_hi[8];
        q4kx8_scales(tile, 2 * g, s_lo, m_lo);
        q4kx8_scales(tile, 2 * g + 1, s_hi, m_hi);
        const __m256i vs_lo = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)s_lo)), vs_hi = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)s_hi));
        const __m256i vm_lo = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)m_lo)), vm_hi = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)m_hi));
        const int b_lo = (int)bs[4 * g] + (int)bs[4 * g + 1], b_hi = (int)bs[4 * g + 2] + (int)bs[4 * g + 3];
        _mm256_storeu_si256((__m256i *)iacc[g], _mm256_add_epi32(_mm256_mullo_epi32(dlo, vs_lo), _mm256_mullo_epi32(dhi, vs_hi)));
        _mm256_storeu_si256((__m256i *)imin[g], _mm256_add_epi32(_mm256_mullo_epi32(vm_lo, _mm256_set1_epi32(b_lo)), _mm256_mullo_epi32(vm_hi, _mm256_set1_epi32(b_hi))));
    }
}

// The same with the 4-byte dot of AVX-512 VNNI on 256-bit registers: no 16-bit intermediate.
__attribute__((target("avx2,avx512f,avx512vl,avx512vnni"))) static void q4kx8_ints_vnni(const uint8_t *tile, const int8_t *q8, const int16_t *bs,
                                                                                        int iacc[4][8], int imin[4][8]) {
    const __m256i m4 = _mm256_set1_epi8(0x0F);
    const __m256i row_order = _mm256_setr_epi32(0, 1, 4, 5, 2, 3, 6, 7);
    for (int g = 0; g < 4; g++) {
        const uint8_t *qs = tile + 128 + 256 * g;
        __m256i lo03 = _mm256_setzero_si256(), lo47 = lo03, hi03 = lo03, hi47 = lo03;
        for (int p = 0; p < 4; p++) {
            const __m256i w03 = _mm256_loadu_si256((const __m256i *)(qs + 64 * p)), w47 = _mm256_loadu_si256((const __m256i *)(qs + 64 * p + 32));
            long long ylo8, yhi8;
            memcpy(&ylo8, q8 + 64 * g + 8 * p, 8);
            memcpy(&yhi8, q8 + 64 * g + 32 + 8 * p, 8);
            const __m256i ylo = _mm256_set1_epi64x(ylo8), yhi = _mm256_set1_epi64x(yhi8);
            lo03 = _mm256_dpbusd_epi32(lo03, _mm256_and_si256(w03, m4), ylo);
            lo47 = _mm256_dpbusd_epi32(lo47, _mm256_and_si256(w47, m4), ylo);
            hi03 = _mm256_dpbusd_epi32(hi03, _mm256_and_si256(_mm256_srli_epi16(w03, 4), m4), yhi);
            hi47 = _mm256_dpbusd_epi32(hi47, _mm256_and_si256(_mm256_srli_epi16(w47, 4), m4), yhi);
        }
        const __m256i dlo = _mm256_permutevar8x32_epi32(_mm256_hadd_epi32(lo03, lo47), row_order);
        const __m256i dhi = _mm256_permutevar8x32_epi32(_mm256_hadd_epi32(hi03, hi47), row_order);
        uint8_t s_lo[8], m_lo[8], s_hi[8], m_hi[8];
        q4kx8_scales(tile, 2 * g, s_lo, m_lo);
        q4kx8_scales(tile, 2 * g + 1, s_hi, m_hi);
        const __m256i vs_lo = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)s_lo)), vs_hi = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)s_hi));
        const __m256i vm_lo = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)m_lo)), vm_hi = _mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i *)m_hi));
        const int b_lo = (int)bs[4 * g] + (int)bs[4 * g + 1], b_hi = (int)bs[4 * g + 2] + (int)bs[4 * g + 3];
        _mm256_storeu_si256((__m256i *)iacc[g], _mm256_add_epi32(_mm256_mullo_epi32(dlo, vs_lo), _mm256_mullo_epi32(dhi, vs_hi)));
        _mm256_storeu_si256((__m256i *)imin[g], _mm256_add_epi32(_mm256_mullo_epi32(vm_lo, _mm256_set1_epi32(b_lo)), _mm256_mullo_epi32(vm_hi, _mm256_set1_epi32(b_hi))));
    }
}

// false: no vector form on this host (or switched off): the caller runs its scalar loop
extern "C" int orc_q4kx8_ints_simd(const uint8_t *tile, const int8_t *q8, const int16_t *bs, int iacc[4][8], int imin[4][8]) {
    const int level = orc_simd_level();
    if (level == 2) { q4kx8_ints_vnni(tile, q8, bs, iacc, imin); return 1; }
    if (level == 1) { q4kx8_ints_avx2(tile, q8, bs, iacc, imin); return 1; }
    return 0;
}

// Q6_K row dot, integer part of one super-block: the eight lane sums of crates/ggml/src/vec_dot.rs:990-1032 (lane l
// collects elements 4 l .. 4 l + 3 of every 32-element run, each product scaled by its 16-element sub-block's scale,
// the -32 bias taken off through the activation's 16-element sums).  ql / qh / sc: the block's fields; q8 / bsums: the
// activation block's.  One 256-bit register holds a 32-element run as bytes; madd with the scale pair (first 16 / last
// 16 elements) replicated per 16-bit lane gives four-element sums in dwords: exactly lane l.
__attribute__((target("avx2"))) static void q6k_lane_sums_avx2(const uint8_t *ql, const uint8_t *qh, const int8_t *sc, const int8_t *q8,
                                                               const int16_t *bsums, int sumi[8]) {
    const __m256i m4 = _mm256_set1_epi8(0x0F), m2 = _mm256_set1_epi8(0x03);
    __m256i acc = _mm256_setzero_si256();
    for (int j = 0; j < 2; j++) {
        const __m256i l0 = _mm256_loadu_si256((const __m256i *)(ql + 64 * j)), l1 = _mm256_loadu_si256((const __m256i *)(ql + 64 * j + 32));
        const __m256i h = _mm256_loadu_si256((const __m256i *)(qh + 32 * j));
        __m256i v[4];
        v[0] = _mm256_or_si256(_mm256_and_si256(l0, m4), _mm256_slli_epi16(_mm256_and_si256(h, m2), 4));
        v[1] = _mm256_or_si256(_mm256_and_si256(l1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 2), m2), 4));
        v[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 4), m2), 4));
        v[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(h, 6), m2), 4));
        for (int k = 0; k < 4; k++) {
            const __m256i y = _mm256_loadu_si256((const __m256i *)(q8 + 128 * j + 32 * k));
            // unsigned 6-bit values x signed quants, adjacent pairs in 16 bits (at most 2 x 63 x 127)
            const __m256i p16 = _mm256_maddubs_epi16(v[k], y);
            // the run's two scales: elements 0..15 (low 128 bits) and 16..31 (high 128 bits)
            const __m256i s16 = _mm256_set_m128i(_mm_set1_epi16(sc[8 * j + 2 * k + 1]), _mm_set1_epi16(sc[8 * j + 2 * k]));
            acc = _mm256_add_epi32(acc, _mm256_madd_epi16(p16, s16));   // dword l = elements 4 l .. 4 l + 3, scaled
        }
    }
    _mm256_storeu_si256((__m256i *)sumi, acc);
    for (int l = 0; l < 8; l++) sumi[l] -= ((int)bsums[2 * l] * (int)sc[2 * l] + (int)bsums[2 * l + 1] * (int)sc[2 * l + 1]) << 5;
}

extern "C" int orc_q6k_lane_sums_simd(const uint8_t *ql, const uint8_t *qh, const int8_t *sc, const int8_t *q8, const int16_t *bsums, int sumi[8]) {
    if (orc_simd_level() < 1) return 0;
    q6k_lane_sums_avx2(ql, qh, sc, q8, bsums, sumi);
    return 1;
}
