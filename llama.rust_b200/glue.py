"""ctypes wrappers of the glue-op entry points of include/ggml_b200.h (RMS_NORM, ADD/MUL, SILU, ROPE,
SET_ROWS, GET_ROWS, ARGMAX).  Host arrays in, host arrays out: every wrapper uploads its operands,
runs the CUDA kernel and reads the result back; nothing is computed on the host except the ROPE
table, which the library itself builds with the host libm (b200_rope_table)."""
import ctypes as C

import numpy as np

from . import DeviceBuffer, check, device_array, lib

vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
lib.b200_rms_norm.argtypes = [vp, i64, vp, i64, vp, vp, i64, i64, i64, f32, vp]
lib.b200_binary.argtypes = [i32, vp, i64, vp, i64, i64, i64, vp, i64, i64, i64, vp]
lib.b200_silu.argtypes = [vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i32, vp]
lib.b200_host_silu_is_wide.restype = i32
lib.b200_rope_table.argtypes = [vp, i64, i64, vp, i32, i32, f32, f32, f32, f32, f32, f32, vp]
lib.b200_rope.argtypes = [vp, i64, i64, vp, i64, i64, vp, vp, i64, i64, i64, i64, i32, i32, vp]
lib.b200_set_rows_f16.argtypes = [vp, i64, vp, vp, i64, i64, i64, i64, vp]
lib.b200_get_rows.argtypes = [i32, vp, i64, i64, vp, i64, vp, i64, vp]
lib.b200_argmax.argtypes = [vp, i64, i64, i64, vp, vp]


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _rows(a):
    return a.size // a.shape[-1]


def rms_norm(x, eps, weight=None):
    """-> y, or (y, y * weight) when weight is given"""
    x = _f(x)
    ne0, n = x.shape[-1], _rows(x)
    dx, dy = device_array(x), DeviceBuffer(x.nbytes)
    dw = device_array(_f(weight)) if weight is not None else None
    dyw = DeviceBuffer(x.nbytes) if weight is not None else None
    check(lib.b200_rms_norm(dx.ptr, ne0, dy.ptr, ne0, dw.ptr if dw else None, dyw.ptr if dyw else None, ne0, ne0, n, eps, None))
    y = dy.download(np.float32, x.size).reshape(x.shape)
    if weight is None:
        return y
    return y, dyw.download(np.float32, x.size).reshape(x.shape)


def binary(op, a, b):
    a, b = _f(a), _f(b)
    ne0 = a.shape[-1]
    da, db, dy = device_array(a), device_array(b), DeviceBuffer(a.nbytes)
    check(lib.b200_binary(op, da.ptr, ne0, db.ptr, b.shape[-1], b.shape[-1], _rows(b), dy.ptr, ne0, ne0, _rows(a), None))
    return dy.download(np.float32, a.size).reshape(a.shape)


def add(a, b):
    return binary(0, a, b)


def mul(a, b):
    return binary(1, a, b)


def silu(x, wide=True, gate=None):
    """-> silu(x), or (silu(x), silu(x) * gate) when gate is given"""
    x = _f(x)
    ne0, n = x.shape[-1], _rows(x)
    dx, dy = device_array(x), DeviceBuffer(x.nbytes)
    dg = device_array(_f(gate)) if gate is not None else None
    dyg = DeviceBuffer(x.nbytes) if gate is not None else None
    check(lib.b200_silu(dx.ptr, ne0, dg.ptr if dg else None, ne0, dy.ptr, ne0, dyg.ptr if dyg else None, ne0, ne0, n, int(wide), None))
    y = dy.download(np.float32, x.size).reshape(x.shape)
    if gate is None:
        return y
    return y, dyg.download(np.float32, x.size).reshape(x.shape)


def rope_table(pos, ne0, n_dims, freq_base=10000.0, freq_scale=1.0, n_ctx_orig=4096, ext_factor=0.0, attn_factor=1.0,
               beta_fast=32.0, beta_slow=1.0, freq_factors=None):
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    table = np.empty((pos.size, ne0), dtype=np.float32)
    ff = None if freq_factors is None else _f(freq_factors)
    check(lib.b200_rope_table(pos.ctypes.data, pos.size, ne0, None if ff is None else ff.ctypes.data, n_dims, n_ctx_orig, freq_base,
                              freq_scale, ext_factor, attn_factor, beta_fast, beta_slow, table.ctypes.data))
    return table


def rope(x, pos, n_dims, mode, by_position_rows=0, **kw):
    """x: [n_tok, n_head, ne0].  by_position_rows > 0: one table of that many positions, indexed by pos on the device."""
    x = _f(x)
    n_tok, n_head, ne0 = x.shape
    if by_position_rows:
        table = rope_table(np.arange(by_position_rows), ne0, n_dims, **kw)
        rows = device_array(np.ascontiguousarray(pos, dtype=np.int32))
    else:
        table, rows = rope_table(pos, ne0, n_dims, **kw), None
    dx, dt, dy = device_array(x), device_array(table), DeviceBuffer(x.nbytes)
    check(lib.b200_rope(dx.ptr, ne0 * 4, n_head * ne0 * 4, dy.ptr, ne0 * 4, n_head * ne0 * 4, dt.ptr, rows.ptr if rows else None,
                        by_position_rows, ne0, n_head, n_tok, n_dims, mode, None))
    return dy.download(np.float32, x.size).reshape(x.shape)


def set_rows_f16(x, idx, dst):
    """rows of f32 x -> rows idx of dst (uint16 f16 bits, [rows, ne0]); returns the new dst"""
    x = _f(x)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    dst = np.ascontiguousarray(dst, dtype=np.uint16)
    ne0 = x.shape[-1]
    dx, di, dd = device_array(x), device_array(idx), device_array(dst)
    check(lib.b200_set_rows_f16(dx.ptr, ne0, di.ptr, dd.ptr, ne0, dst.shape[0], ne0, _rows(x), None))
    return dd.download(np.uint16, dst.size).reshape(dst.shape)


def get_rows(ty, table_ptr, ne0, table_rows, ids):
    """table_ptr: device pointer of a dense F32/F16 table or of a Weight's tiles"""
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    di, dy = device_array(ids), DeviceBuffer(ids.size * ne0 * 4)
    check(lib.b200_get_rows(ty, table_ptr, ne0, table_rows, di.ptr, ids.size, dy.ptr, ne0, None))
    return dy.download(np.float32, ids.size * ne0).reshape(ids.size, ne0)


def argmax(x):
    x = _f(x)
    x2 = x.reshape(-1, x.shape[-1])
    dx, do = device_array(x2), DeviceBuffer(x2.shape[0] * 4)
    check(lib.b200_argmax(dx.ptr, x2.shape[1], x2.shape[1], x2.shape[0], do.ptr, None))
    return do.download(np.int32, x2.shape[0])


lib.b200_rms_norm_q8.argtypes = [vp, i64, vp, i64, vp, vp, i64, i64, i64, f32, vp, i32, vp]
lib.b200_silu_q8.argtypes = [vp, i64, vp, i64, vp, i64, vp, i64, i64, i64, i32, vp, i32, vp]


def _read_q8_K(dact, m, k):
    """(qs int8 [m, k], d f32 [m, k/256], bsums i16 [m, k/16]) out of a device activation scratch"""
    def up(v):
        return (v + 255) // 256 * 256
    o_d = up(m * k)
    o_b = o_d + up(m * (k // 256) * 4)
    qs = dact.download(np.int8, m * k).reshape(m, k)
    d = dact.download(np.float32, m * (k // 256), offset=o_d).reshape(m, k // 256)
    bs = dact.download(np.int16, m * (k // 16), offset=o_b).reshape(m, k // 16)
    return qs, d, bs


def rms_norm_q8(x, eps, weight, act_kind):
    """-> (y, y * weight, (qs, d, bsums) of y * weight)"""
    x = _f(x)
    ne0, n = x.shape[-1], _rows(x)
    dx, dy, dyw, dw = device_array(x), DeviceBuffer(x.nbytes), DeviceBuffer(x.nbytes), device_array(_f(weight))
    dact = DeviceBuffer(lib.b200_act_scratch_nbytes(n, ne0))
    check(lib.b200_rms_norm_q8(dx.ptr, ne0, dy.ptr, ne0, dw.ptr, dyw.ptr, ne0, ne0, n, eps, dact.ptr, act_kind, None))
    return (dy.download(np.float32, x.size).reshape(x.shape), dyw.download(np.float32, x.size).reshape(x.shape),
            _read_q8_K(dact, n, ne0))


def silu_q8(x, gate, wide, act_kind):
    """-> (silu(x), silu(x) * gate, (qs, d, bsums) of the product)"""
    x, gate = _f(x), _f(gate)
    ne0, n = x.shape[-1], _rows(x)
    dx, dg, dy, dyg = device_array(x), device_array(gate), DeviceBuffer(x.nbytes), DeviceBuffer(x.nbytes)
    dact = DeviceBuffer(lib.b200_act_scratch_nbytes(n, ne0))
    check(lib.b200_silu_q8(dx.ptr, ne0, dg.ptr, ne0, dy.ptr, ne0, dyg.ptr, ne0, ne0, n, int(wide), dact.ptr, act_kind, None))
    return (dy.download(np.float32, x.size).reshape(x.shape), dyg.download(np.float32, x.size).reshape(x.shape),
            _read_q8_K(dact, n, ne0))
