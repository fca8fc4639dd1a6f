// Quantized tensors on the device: ggml block order <-> 32-row tile layout, and
// dequantization straight from the tile layout.
//
// The tile layout plays the role of the CPU path's load-time CPU_REPACK
// interleave (crates/ggml/src/repack.rs:165,1435,3260): same bytes, re-ordered
// once at upload.  b200_weight_download() is its exact inverse, and
// b200_dequantize() must reproduce dequantize_row (crates/ggml/src/quants.rs:1098)
// bit for bit through it.
#include "common.cuh"

namespace b200 {

// position of (row, src byte) inside a (tile, group) chunk: inverse of chunk_byte_to_src
__host__ __device__ inline int src_to_chunk_byte(int type, int row, int src) {
    switch (type) {
        case B200_TYPE_Q4_K:
            if (src < 16) return row * 16 + src;
            return 512 + ((src - 16) / 16) * 512 + row * 16 + (src - 16) % 16;
        case B200_TYPE_Q6_K:
            if (src < 128) return (src / 16) * 512 + row * 16 + src % 16;
            if (src < 192) return 4096 + ((src - 128) / 16) * 512 + row * 16 + (src - 128) % 16;
            if (src < 208) return 6144 + row * 16 + (src - 192);
            return 6656 + row * 2 + (src - 208);
        case B200_TYPE_Q8_0: {
            int blk = src / 34, o = src % 34;
            if (o < 2) return 8192 + row * 16 + blk * 2 + o;
            return (blk * 2 + (o - 2) / 16) * 512 + row * 16 + (o - 2) % 16;
        }
        case B200_TYPE_Q4_0: {
            int blk = src / 18, o = src % 18;
            if (o < 2) return 4096 + row * 16 + blk * 2 + o;
            return blk * 512 + row * 16 + (o - 2);
        }
        case B200_TYPE_MXFP4: {
            int blk = src / 17, o = src % 17;
            if (o == 0) return 4096 + row * 8 + blk;
            return blk * 512 + row * 16 + (o - 1);
        }
        default: return 0;
    }
}

// One thread per tile byte.  forward: tiles[p] = blocks[src(p)] (0 for pad rows);
// inverse: blocks[src(p)] = tiles[p].
__global__ void repack_kernel(int type, int64_t n_rows, int64_t groups, int gsb, int cb, const uint8_t *src,
                              uint8_t *dst, bool inverse, int64_t total) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    int64_t chunk = i / cb;
    int p = (int)(i % cb);
    int64_t tile = chunk / groups, g = chunk % groups;
    int r, s;
    chunk_byte_to_src(type, p, &r, &s);
    int64_t row = tile * TILE_ROWS + r;
    int64_t plain = (row * groups + g) * gsb + s;
    if (!inverse) {
        dst[i] = row < n_rows ? src[plain] : (uint8_t)0;
    } else if (row < n_rows) {
        dst[plain] = src[i];
    }
}

int launch_repack(int type, int64_t n_rows, int64_t k, const uint8_t *src, uint8_t *dst, bool inverse,
                  cudaStream_t s) {
    const int gsb = group_src_bytes(type);
    B200_REQUIRE(gsb != 0, "repack: type %d is not a supported quantized type", type);
    B200_REQUIRE(k > 0 && k % GROUP_K == 0, "repack: k = %lld must be a positive multiple of 256", (long long)k);
    if (n_rows == 0) return B200_STATUS_SUCCESS;
    const int64_t groups = k / GROUP_K;
    const int64_t tiles = (n_rows + TILE_ROWS - 1) / TILE_ROWS;
    const int cb = chunk_bytes(type);
    const int64_t total = tiles * groups * cb;
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    B200_REQUIRE(blocks < 0x7fffffffLL, "repack: tensor too large for one launch");
    repack_kernel<<<(unsigned)blocks, threads, 0, s>>>(type, n_rows, groups, gsb, cb, src, dst, inverse, total);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

// ---- dequantize --------------------------------------------------------------
__device__ __forceinline__ uint8_t tb(const uint8_t *chunk, int type, int row, int src) {
    return chunk[src_to_chunk_byte(type, row, src)];
}
__device__ __forceinline__ float th(const uint8_t *chunk, int type, int row, int src) {
    uint16_t h = (uint16_t)tb(chunk, type, row, src) | ((uint16_t)tb(chunk, type, row, src + 1) << 8);
    return f16_bits_to_f32(h);
}

__constant__ int8_t c_kvalues_mxfp4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

// One thread per element.  Every product/sum is an explicit round-to-nearest
// op so that nothing is contracted into an FMA the CPU path does not have.
__device__ float dequantize_element(int type, int64_t k, const uint8_t *tiles, int64_t row, int64_t col) {
    const int64_t groups = k / GROUP_K;
    const int64_t tile = row / TILE_ROWS;
    const int r = (int)(row % TILE_ROWS);
    const int64_t g = col / GROUP_K;
    const int e = (int)(col % GROUP_K);
    const uint8_t *c = tiles + (tile * groups + g) * (int64_t)chunk_bytes(type);
    float v = 0.0f;
    switch (type) {
        case B200_TYPE_Q4_K: {  // crates/ggml/src/quants.rs:519-547
            const float d = th(c, type, r, 0), dmin = th(c, type, r, 2);
            const int j = e / 32;  // sub-block 0..7
            uint8_t sc, m;
            if (j < 4) {
                sc = tb(c, type, r, 4 + j) & 63;
                m = tb(c, type, r, 4 + j + 4) & 63;
            } else {
                sc = (tb(c, type, r, 4 + j + 4) & 0xF) | ((tb(c, type, r, 4 + j - 4) >> 6) << 4);
                m = (tb(c, type, r, 4 + j + 4) >> 4) | ((tb(c, type, r, 4 + j) >> 6) << 4);
            }
            const uint8_t qb = tb(c, type, r, 16 + 32 * (e / 64) + e % 32);
            const int q = (j & 1) ? (qb >> 4) : (qb & 0xF);
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
            break;
        }
        case B200_TYPE_Q6_K: {  // crates/ggml/src/quants.rs:585-612
            const float d = th(c, type, r, 208);
            const int n = e / 128, rr = e % 128, kk = rr / 32, l = rr % 32;
            const uint8_t qlb = tb(c, type, r, 64 * n + (kk & 1) * 32 + l);
            const uint8_t qhb = tb(c, type, r, 128 + 32 * n + l);
            const int nib = (kk >= 2) ? (qlb >> 4) : (qlb & 0xF);
            const int q = (int)(int8_t)(nib | (((qhb >> (2 * kk)) & 3) << 4)) - 32;
            const int8_t sc = (int8_t)tb(c, type, r, 192 + 8 * n + l / 16 + 2 * kk);
            v = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
            break;
        }
        case B200_TYPE_Q8_0: {  // crates/ggml/src/quants.rs:364-373
            const int blk = e / 32, j = e % 32;
            v = __fmul_rn((float)(int8_t)tb(c, type, r, 34 * blk + 2 + j), th(c, type, r, 34 * blk));
            break;
        }
        case B200_TYPE_Q4_0: {  // crates/ggml/src/quants.rs:154-167
            const int blk = e / 32, j = e % 32;
            const uint8_t qb = tb(c, type, r, 18 * blk + 2 + j % 16);
            const int q = (j < 16 ? (qb & 0xF) : (qb >> 4)) - 8;
            v = __fmul_rn((float)q, th(c, type, r, 18 * blk));
            break;
        }
        case B200_TYPE_MXFP4: {  // crates/ggml/src/quants.rs:732-746
            const int blk = e / 32, j = e % 32;
            const uint8_t qb = tb(c, type, r, 17 * blk + 1 + j % 16);
            const int q = c_kvalues_mxfp4[j < 16 ? (qb & 0xF) : (qb >> 4)];
            v = __fmul_rn((float)q, e8m0_half_to_f32(tb(c, type, r, 17 * blk)));
            break;
        }
        default: break;
    }
    return v;
}

__global__ void dequantize_kernel(int type, int64_t n_rows, int64_t k, const uint8_t *tiles, float *out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows * k) return;
    out[i] = dequantize_element(type, k, tiles, i / k, i % k);
}

// GET_ROWS over a tiled table (crates/ggml/src/compute.rs:3842-3895): row ids[r] to f32, one
// thread per element; an id outside the table leaves the row untouched and raises the error flag.
__global__ void get_rows_tiled_kernel(int type, int64_t table_rows, int64_t k, const uint8_t *tiles, const int32_t *ids,
                                      int64_t n, float *out, int64_t out_stride, int *err) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * k) return;
    const int64_t r = i / k, col = i % k;
    const int64_t row = ids[r];
    if (row < 0 || row >= table_rows) {
        if (col == 0) atomicExch(err, 1);
        return;
    }
    out[r * out_stride + col] = dequantize_element(type, k, tiles, row, col);
}

int launch_dequantize(int type, int64_t n_rows, int64_t k, const uint8_t *tiles, float *out, cudaStream_t s) {
    B200_REQUIRE(group_src_bytes(type) != 0, "dequantize: type %d is not a supported quantized type", type);
    B200_REQUIRE(k > 0 && k % GROUP_K == 0, "dequantize: k = %lld must be a positive multiple of 256", (long long)k);
    if (n_rows == 0) return B200_STATUS_SUCCESS;
    const int64_t total = n_rows * k;
    const int threads = 256;
    const int64_t blocks = (total + threads - 1) / threads;
    B200_REQUIRE(blocks < 0x7fffffffLL, "dequantize: tensor too large for one launch");
    dequantize_kernel<<<(unsigned)blocks, threads, 0, s>>>(type, n_rows, k, tiles, out);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

int launch_get_rows_tiled(int type, int64_t table_rows, int64_t k, const uint8_t *tiles, const int32_t *ids, int64_t n,
                          float *out, int64_t out_stride, int *err, cudaStream_t s) {
    B200_REQUIRE(group_src_bytes(type) != 0, "get_rows: type %d is not a supported quantized type", type);
    B200_REQUIRE(k > 0 && k % GROUP_K == 0, "get_rows: k = %lld must be a positive multiple of 256", (long long)k);
    if (n == 0) return B200_STATUS_SUCCESS;
    const int threads = 256;
    const int64_t blocks = (n * k + threads - 1) / threads;
    B200_REQUIRE(blocks < 0x7fffffffLL, "get_rows: too many rows for one launch");
    get_rows_tiled_kernel<<<(unsigned)blocks, threads, 0, s>>>(type, table_rows, k, tiles, ids, n, out, out_stride, err);
    B200_CUDA(cudaGetLastError());
    return B200_STATUS_SUCCESS;
}

}  // namespace b200
