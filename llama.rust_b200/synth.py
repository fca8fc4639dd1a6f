"""Synthetic quantized tensors for benchmarks: random but well-formed ggml blocks, made with numpy alone.

Timing does not depend on the weight values, so a benchmark does not need a real quantizer: every
block below decodes to finite weights of roughly N(0, 0.05) spread (uniform quants times a small
scale), which keeps a random-init decoder's activations finite through any number of layers.  Large
matrices repeat `period` distinct rows.  (Tests that compare values quantize real f32 data with the
CPU oracle instead.)"""
import numpy as np

# ggml type ids (this module imports nothing of the package at load time: a CPU-only process can load it by path)
F32, Q4_0, Q8_0, Q4_K, Q6_K, MXFP4 = 0, 2, 8, 12, 14, 39

BLOCK = {Q4_K: (256, 144), Q6_K: (256, 210), Q8_0: (32, 34), Q4_0: (32, 18), MXFP4: (32, 17)}


def _f16_bytes(rng, lo, hi, n):
    return rng.uniform(lo, hi, n).astype(np.float16).view(np.uint8).reshape(n, 2)


def blocks(ty, rows, ne0, seed=0, period=4096):
    """uint8 [rows, row_bytes] of ggml blocks of type ty"""
    per, size = BLOCK[ty]
    assert ne0 % per == 0
    nb = ne0 // per
    distinct = min(rows, period)
    rng = np.random.default_rng(seed)
    n = distinct * nb
    b = rng.integers(0, 256, (n, size), dtype=np.uint8)
    if ty == Q4_K:        # d, dmin, scales[12], qs[128]
        b[:, 0:2] = _f16_bytes(rng, 1.5e-4, 4.5e-4, n)
        b[:, 2:4] = _f16_bytes(rng, 1.2e-3, 3.7e-3, n)
    elif ty == Q6_K:      # ql[128], qh[64], scales[16] (i8), d
        b[:, 192:208] = rng.integers(-32, 33, (n, 16)).astype(np.int8).view(np.uint8)
        b[:, 208:210] = _f16_bytes(rng, 0.8e-4, 2.4e-4, n)
    elif ty == Q8_0:      # d, qs[32] (i8)
        b[:, 0:2] = _f16_bytes(rng, 3e-4, 9e-4, n)
    elif ty == Q4_0:      # d, qs[16]
        b[:, 0:2] = _f16_bytes(rng, 5e-3, 1.5e-2, n)
    elif ty == MXFP4:     # e (E8M0), qs[16]
        b[:, 0] = rng.integers(118, 122, n, dtype=np.uint8)
    q = b.reshape(distinct, nb * size)
    if distinct < rows:
        q = np.tile(q, ((rows + distinct - 1) // distinct, 1))[:rows]
    return np.ascontiguousarray(q)


def llama_tensors(hp, type_of, seed=0, period=4096, tensor_shapes=None):
    """yields (name, type, array, ne0, ne1) for every tensor of a llama-architecture model"""
    if tensor_shapes is None:
        from .shapes import tensor_shapes
    rng = np.random.default_rng(seed)
    for i, (name, (ne0, ne1)) in enumerate(tensor_shapes(hp).items()):
        ty = type_of(name)
        if ty == F32:
            yield name, ty, (1.0 + 0.1 * rng.standard_normal(ne0)).astype(np.float32), ne0, ne1
        else:
            yield name, ty, blocks(ty, ne1, ne0, seed=seed * 100003 + i, period=period), ne0, ne1
