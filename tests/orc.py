"""ctypes binding of the CPU oracle (oracle/liboracle.so) for the tests.

The oracle is test infrastructure: it restates the reference's CPU arithmetic
and is the checker the CUDA path is compared against.  Nothing here is used by
the shipped library.
"""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, Q8_K, MXFP4 = 0, 1, 2, 8, 12, 14, 15, 39
TYPE_NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", MXFP4: "MXFP4", Q8_K: "Q8_K"}
ROUTE_AUTO, ROUTE_ROWDOT, ROUTE_REPACK, ROUTE_TILED = 0, 1, 2, 3

_lib = None


def build():
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)


def lib():
    global _lib
    if _lib is not None:
        return _lib
    path = os.path.join(ORACLE_DIR, "liboracle.so")
    if not os.path.exists(path):
        build()
    L = C.CDLL(path)
    vp, i64, i32, f32p = C.c_void_p, C.c_int64, C.c_int, C.POINTER(C.c_float)
    L.orc_f32_to_f16.restype = C.c_uint16
    L.orc_f32_to_f16.argtypes = [C.c_float]
    L.orc_f16_to_f32.restype = C.c_float
    L.orc_f16_to_f32.argtypes = [C.c_uint16]
    L.orc_row_size.restype = C.c_size_t
    L.orc_row_size.argtypes = [i32, i64]
    L.orc_quantize_row.argtypes = [i32, vp, vp, i64]
    L.orc_dequantize_row.argtypes = [i32, vp, vp, i64]
    L.orc_quantize_rows.argtypes = [i32, vp, vp, i64, i64]
    L.orc_quantize_row_q8_0.argtypes = [vp, vp, i64]
    L.orc_quantize_row_q8_K.argtypes = [vp, vp, i64]
    L.orc_quantize_mat_q8_K_4x8.argtypes = [vp, i64, i64, vp]
    L.orc_quantize_mat_q8_0_4x8.argtypes = [vp, i64, i64, vp]
    L.orc_repack_8x8.argtypes = [i32, vp, i64, i64, vp]
    L.orc_vec_dot.restype = C.c_float
    L.orc_vec_dot.argtypes = [i32, i64, vp, vp]
    L.orc_gemv_8x8.argtypes = [i32, i64, vp, vp, vp, i64]
    L.orc_gemm_8x8.argtypes = [i32, i64, vp, i64, vp, vp, i64, i64]
    L.orc_mul_mat.argtypes = [i32, i64, i64, i64, vp, vp, vp, i32, i32]
    L.orc_mul_mat_repacked.argtypes = [i32, i64, i64, i64, vp, vp, vp, i32]
    L.orc_mul_mat_id.argtypes = [i32, i64, i64, i64, i64, i64, i64, vp, vp, vp, vp, i32, i32]
    L.orc_flash_attn_ext.argtypes = [vp]
    L.orc_set_simd.restype = None
    L.orc_set_simd.argtypes = [i32]
    L.orc_simd_level.restype = i32
    _lib = L
    return L


def set_simd(max_level):
    """Caps the oracle's vector level: 0 scalar, 1 AVX2, 2 AVX-512 VNNI."""
    lib().orc_set_simd(max_level)


def simd_level():
    return lib().orc_simd_level()


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def row_size(ty, k):
    return lib().orc_row_size(ty, k)


def quantize(ty, x):
    """x: f32 [rows, k] (or [k]) -> uint8 [rows, row_size]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    x2 = x.reshape(-1, x.shape[-1])
    rows, k = x2.shape
    rs = row_size(ty, k)
    out = np.zeros((rows, rs), dtype=np.uint8)
    for r in range(rows):
        rc = lib().orc_quantize_row(ty, _p(x2[r]), _p(out[r]), k)
        assert rc == 0
    return out.reshape(x.shape[:-1] + (rs,))


def quantize_rows(ty, x):
    """x: f32 [rows, k] -> uint8 [rows, row_size], rows spread over the host threads."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    out = np.zeros((rows, row_size(ty, k)), dtype=np.uint8)
    assert lib().orc_quantize_rows(ty, _p(x), _p(out), rows, k) == 0
    return out


def dequantize(ty, q, k):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    q2 = q.reshape(-1, q.shape[-1])
    out = np.zeros((q2.shape[0], k), dtype=np.float32)
    for r in range(q2.shape[0]):
        rc = lib().orc_dequantize_row(ty, _p(q2[r]), _p(out[r]), k)
        assert rc == 0
    return out.reshape(q.shape[:-1] + (k,))


def quantize_q8_0(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    rows = x.size // k
    out = np.zeros((rows, k // 32 * 34), dtype=np.uint8)
    lib().orc_quantize_row_q8_0(_p(x), _p(out), rows * k)
    return out


def quantize_q8_K(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    k = x.shape[-1]
    rows = x.size // k
    out = np.zeros((rows, k // 256 * 292), dtype=np.uint8)
    lib().orc_quantize_row_q8_K(_p(x), _p(out), rows * k)
    return out


def quantize_q8_K_4x8(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    out = np.zeros((rows // 4) * (k // 256) * 1168, dtype=np.uint8)
    lib().orc_quantize_mat_q8_K_4x8(_p(x), k, rows, _p(out))
    return out


def quantize_q8_0_4x8(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, k = x.shape
    out = np.zeros((rows // 4) * (k // 32) * 136, dtype=np.uint8)
    lib().orc_quantize_mat_q8_0_4x8(_p(x), k, rows, _p(out))
    return out


def repack_8x8(ty, w, nrows, k):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    out = np.zeros(w.size, dtype=np.uint8)
    rc = lib().orc_repack_8x8(ty, _p(w), nrows, k, _p(out))
    assert rc == 0
    return out


def gemv_8x8(ty, k, vx, vy, nc):
    out = np.zeros(nc, dtype=np.float32)
    rc = lib().orc_gemv_8x8(ty, k, _p(out), _p(np.ascontiguousarray(vx)), _p(np.ascontiguousarray(vy)), nc)
    assert rc == 0
    return out


def gemm_8x8(ty, k, vx, vy, nr, nc):
    out = np.zeros((nr, nc), dtype=np.float32)
    rc = lib().orc_gemm_8x8(ty, k, _p(out), nc, _p(np.ascontiguousarray(vx)), _p(np.ascontiguousarray(vy)), nr, nc)
    assert rc == 0
    return out


def vec_dot(ty, k, w_row, a_row):
    return lib().orc_vec_dot(ty, k, _p(np.ascontiguousarray(w_row)), _p(np.ascontiguousarray(a_row)))


def mul_mat(ty, W, X, route=ROUTE_AUTO, n_threads=0):
    """W: uint8 [N, row_size]; X: f32 [M, K] -> (out f32 [M, N], route taken)."""
    W = np.ascontiguousarray(W, dtype=np.uint8)
    X = np.ascontiguousarray(X, dtype=np.float32)
    N = W.shape[0]
    M, K = X.shape
    assert W.shape[1] == row_size(ty, K)
    out = np.zeros((M, N), dtype=np.float32)
    r = lib().orc_mul_mat(ty, N, K, M, _p(W), _p(X), _p(out), route, n_threads)
    assert r > 0, f"orc_mul_mat failed ({r})"
    return out, r


def mul_mat_id(ty, W, B, ids, route=ROUTE_AUTO, n_threads=0):
    """W: uint8 [E, N, row_size]; B: f32 [n_tok, ne11, K]; ids: i32 [n_tok, n_ids]
    -> out f32 [n_tok, n_ids, N]."""
    W = np.ascontiguousarray(W, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    E, N, _ = W.shape
    n_tok, ne11, K = B.shape
    n_ids = ids.shape[1]
    out = np.zeros((n_tok, n_ids, N), dtype=np.float32)
    r = lib().orc_mul_mat_id(ty, N, K, E, ne11, n_tok, n_ids, _p(W), _p(B), _p(ids), _p(out), route, n_threads)
    assert r > 0, f"orc_mul_mat_id failed ({r})"
    return out, r


class FlashArgs(C.Structure):
    _fields_ = [
        ("dk", C.c_int64), ("dv", C.c_int64), ("T", C.c_int64), ("H", C.c_int64),
        ("H_kv", C.c_int64), ("n_kv", C.c_int64),
        ("q", C.c_void_p), ("q_nb1", C.c_int64), ("q_nb2", C.c_int64),
        ("k", C.c_void_p), ("k_nb1", C.c_int64), ("k_nb2", C.c_int64),
        ("v", C.c_void_p), ("v_nb1", C.c_int64), ("v_nb2", C.c_int64),
        ("mask", C.c_void_p), ("mask_nb1", C.c_int64),
        ("sinks", C.c_void_p),
        ("scale", C.c_float), ("max_bias", C.c_float), ("logit_softcap", C.c_float),
        ("dst", C.c_void_p),
        ("mode", C.c_int), ("n_chunks", C.c_int), ("n_threads", C.c_int),
    ]


FA_AUTO, FA_ONE_CHUNK, FA_SPLIT_KV, FA_TILED = 0, 1, 2, 3


def flash_attn(q, k, v, mask, scale, sinks=None, max_bias=0.0, softcap=0.0, mode=FA_AUTO, n_chunks=8,
               n_threads=0):
    """q: f32 [H, T, DK]; k: f16(bits uint16) [H_kv, n_kv, DK]; v: [H_kv, n_kv, DV];
    mask: f16 bits [T, n_kv] or None -> dst f32 [T, H, DV].  (ggml ne order is
    the reverse of these numpy shapes.)"""
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    H, T, DK = q.shape
    H_kv, n_kv, _ = k.shape
    DV = v.shape[2]
    dst = np.zeros((T, H, DV), dtype=np.float32)
    a = FlashArgs()
    a.dk, a.dv, a.T, a.H, a.H_kv, a.n_kv = DK, DV, T, H, H_kv, n_kv
    a.q, a.q_nb1, a.q_nb2 = q.ctypes.data, DK * 4, T * DK * 4
    a.k, a.k_nb1, a.k_nb2 = k.ctypes.data, DK * 2, n_kv * DK * 2
    a.v, a.v_nb1, a.v_nb2 = v.ctypes.data, DV * 2, n_kv * DV * 2
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint16)
        a.mask, a.mask_nb1 = mask.ctypes.data, n_kv * 2
    else:
        a.mask, a.mask_nb1 = None, 0
    if sinks is not None:
        sinks = np.ascontiguousarray(sinks, dtype=np.float32)
        a.sinks = sinks.ctypes.data
    else:
        a.sinks = None
    a.scale, a.max_bias, a.logit_softcap = scale, max_bias, softcap
    a.dst = dst.ctypes.data
    a.mode, a.n_chunks, a.n_threads = mode, n_chunks, n_threads
    rc = lib().orc_flash_attn_ext(C.byref(a))
    assert rc > 0, f"orc_flash_attn_ext failed ({rc})"
    return dst, rc
