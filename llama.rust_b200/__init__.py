"""ctypes binding of libggml-b200.so (the C ABI in include/ggml_b200.h).

This package holds no compute of its own: every call goes straight into the
CUDA library, and importing it fails loudly when the library has not been
built.  The directory name contains a dot, so load it by path:

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("llama_rust_b200", "<repo>/llama.rust_b200/__init__.py")
    mod = importlib.util.module_from_spec(spec); sys.modules["llama_rust_b200"] = mod
    spec.loader.exec_module(mod)
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libggml-b200.so")

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K, Q8_K, MXFP4 = 0, 1, 2, 8, 12, 14, 15, 39
ACT_Q8_0, ACT_Q8_K, ACT_Q8_K_4X8, ACT_Q8_K_MIXED = 1, 2, 3, 4
ROUTE_AUTO, ROUTE_ROWDOT, ROUTE_REPACK, ROUTE_TILED = 0, 1, 2, 3
STATUS_SUCCESS = 0

# bytes per 256 elements of one row, in ggml block order
GROUP_BYTES = {Q4_K: 144, Q6_K: 210, Q8_0: 8 * 34, Q4_0: 8 * 18, MXFP4: 8 * 17}


class B200Error(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise B200Error(f"{LIB_PATH} is missing: build it with `python llama.rust_b200/build.py`")
    L = C.CDLL(LIB_PATH)
    vp, i64, i32, sz = C.c_void_p, C.c_int64, C.c_int, C.c_size_t
    L.b200_last_error.restype = C.c_char_p
    L.b200_device_count.restype = i32
    L.b200_set_device.argtypes = [i32]
    L.b200_device_info.argtypes = [i32, C.c_char_p, sz, C.POINTER(sz), C.POINTER(sz), C.POINTER(i32),
                                   C.POINTER(i32), C.POINTER(i32)]
    L.b200_synchronize.argtypes = [vp]
    L.b200_malloc.argtypes = [C.POINTER(vp), sz]
    L.b200_free.argtypes = [vp]
    L.b200_memcpy_h2d.argtypes = [vp, vp, sz, vp]
    L.b200_memcpy_d2h.argtypes = [vp, vp, sz, vp]
    L.b200_memset.argtypes = [vp, i32, sz, vp]
    L.b200_host_alloc_pinned.argtypes = [C.POINTER(vp), sz]
    L.b200_host_free_pinned.argtypes = [vp]
    L.b200_weight_nbytes.restype = sz
    L.b200_weight_nbytes.argtypes = [i32, i64, i64]
    L.b200_weight_upload.argtypes = [i32, i64, i64, vp, vp, vp]
    L.b200_weight_download.argtypes = [i32, i64, i64, vp, vp, vp]
    L.b200_dequantize.argtypes = [i32, i64, i64, vp, vp, vp]
    L.b200_quantize_activations.argtypes = [i32, i64, i64, vp, vp, vp]
    L.b200_act_scratch_nbytes.restype = sz
    L.b200_act_scratch_nbytes.argtypes = [i64, i64]
    L.b200_quantize_activations_device.argtypes = [i32, i64, i64, vp, i64, vp, vp]
    L.b200_mul_mat_q8.argtypes = [i32, i64, i64, i64, vp, vp, i32, vp, i64, i32, vp]
    L.b200_event_create.argtypes = [C.POINTER(vp)]
    L.b200_event_destroy.argtypes = [vp]
    L.b200_event_record.argtypes = [vp, vp]
    L.b200_event_synchronize.argtypes = [vp]
    L.b200_event_elapsed_ms.argtypes = [vp, vp, C.POINTER(C.c_float)]
    L.b200_mul_mat.argtypes = [i32, i64, i64, i64, vp, vp, i64, vp, i64, i32, vp]
    L.b200_static_scratch_nbytes.restype = sz
    L.b200_mul_mat_static_scratch.argtypes = [i32, i64, i64, i64, vp, vp, i64, vp, i64, i32, vp]
    L.b200_mul_mat_host.argtypes = [i32, i64, i64, i64, vp, vp, vp, i32, vp]
    L.b200_mul_mat_id.argtypes = [i32, i64, i64, i64, i64, i64, i64, vp, vp, vp, vp, i32, vp]
    L.b200_flash_attn_ext.argtypes = [vp, vp]
    L.b200_bench_mul_mat_q8.argtypes = [i32, i64, i64, i64, C.POINTER(vp), i32, vp, i32, vp, i32, C.POINTER(C.c_float)]
    L.b200_set_numerics.argtypes = [i32]
    L.b200_set_numerics.restype = None
    L.b200_debug_alloc_count.restype = C.c_ulonglong
    L.b200_debug_stream_wait.argtypes = [i32, i32]
    L.b200_debug_stream_wait.restype = None
    L.b200_debug_gemm_fast_wait.argtypes = [i32, i32]
    L.b200_debug_gemm_fast_wait.restype = None
    L.b200_debug_rows_ring_wait.argtypes = [i32, i32]
    L.b200_debug_rows_ring_wait.restype = None
    L.b200_debug_decode_step_launches.restype = C.c_ulonglong
    L.b200_debug_decode_step_wait.argtypes = [i32, i32, i32]
    L.b200_debug_decode_step_wait.restype = None
    return L


lib = _load()


def check(rc, what=""):
    if rc != STATUS_SUCCESS:
        raise B200Error(f"{what}: status {rc}: {lib.b200_last_error().decode()}")


def device_count():
    return lib.b200_device_count()


def set_device(i):
    check(lib.b200_set_device(i), "set_device")


def synchronize(stream=None):
    check(lib.b200_synchronize(stream), "synchronize")


EXACT, FAST = 0, 1


def set_numerics(mode):
    """EXACT: bit-exact reproduction of the CPU routes; FAST: tolerance-mode kernels where they exist"""
    lib.b200_set_numerics(mode)


def get_numerics():
    return lib.b200_get_numerics()


def kernel_error():
    """Code left by a kernel whose bounded wait ran out (0 = none); cleared by the read."""
    code = C.c_int(0)
    check(lib.b200_kernel_error(C.byref(code)), "kernel_error")
    return code.value


class DeviceBuffer:
    """A cudaMalloc allocation owned by Python."""

    def __init__(self, nbytes):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        check(lib.b200_malloc(C.byref(p), max(self.nbytes, 1)), "malloc")
        self.ptr = p.value

    def upload(self, arr, offset=0, stream=None):
        arr = np.ascontiguousarray(arr)
        assert offset + arr.nbytes <= self.nbytes
        check(lib.b200_memcpy_h2d(self.ptr + offset, arr.ctypes.data, arr.nbytes, stream), "h2d")
        synchronize(stream)
        return self

    def download(self, dtype, count, offset=0, stream=None):
        out = np.empty(count, dtype=dtype)
        assert offset + out.nbytes <= self.nbytes
        check(lib.b200_memcpy_d2h(out.ctypes.data, self.ptr + offset, out.nbytes, stream), "d2h")
        return out

    def free(self):
        if self.ptr:
            lib.b200_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def device_array(arr):
    arr = np.ascontiguousarray(arr)
    return DeviceBuffer(arr.nbytes).upload(arr)


class Weight:
    """A quantized [n_rows, k] tensor resident on the device in tile layout."""

    def __init__(self, ty, blocks, k):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        self.ty, self.k = ty, int(k)
        self.row_bytes = self.k // 256 * GROUP_BYTES[ty]
        self.n_rows = blocks.size // self.row_bytes
        assert blocks.size == self.n_rows * self.row_bytes
        nbytes = lib.b200_weight_nbytes(ty, self.n_rows, self.k)
        if nbytes == 0 and self.n_rows:
            raise B200Error(f"unsupported weight shape type={ty} rows={self.n_rows} k={k}")
        self.buf = DeviceBuffer(nbytes)
        check(lib.b200_weight_upload(ty, self.n_rows, self.k, blocks.ctypes.data, self.buf.ptr, None), "weight_upload")

    @property
    def ptr(self):
        return self.buf.ptr

    def download(self):
        out = np.empty((self.n_rows, self.row_bytes), dtype=np.uint8)
        check(lib.b200_weight_download(self.ty, self.n_rows, self.k, self.buf.ptr, out.ctypes.data, None),
              "weight_download")
        return out

    def dequantize(self):
        out = DeviceBuffer(self.n_rows * self.k * 4)
        check(lib.b200_dequantize(self.ty, self.n_rows, self.k, self.buf.ptr, out.ptr, None), "dequantize")
        return out.download(np.float32, self.n_rows * self.k).reshape(self.n_rows, self.k)


def quantize_activations(kind, x):
    """x f32 [m, k] -> the CPU path's block bytes (uint8, flat)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    dx = device_array(x)
    if kind == ACT_Q8_0:
        nbytes = m * (k // 32) * 34
    elif kind == ACT_Q8_K:
        nbytes = m * (k // 256) * 292
    else:
        nbytes = (m // 4) * (k // 256) * 1168
    out = np.zeros(nbytes, dtype=np.uint8)
    check(lib.b200_quantize_activations(kind, m, k, dx.ptr, out.ctypes.data, None), "quantize_activations")
    return out


def mul_mat(w, x, route=ROUTE_AUTO):
    """w: Weight [n, k]; x: f32 [m, k] host -> f32 [m, n] through the host-buffer entry point."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, k = x.shape
    assert k == w.k
    out = np.empty((m, w.n_rows), dtype=np.float32)
    check(lib.b200_mul_mat_host(w.ty, w.n_rows, k, m, w.ptr, x.ctypes.data, out.ctypes.data, route, None), "mul_mat_host")
    return out


def mul_mat_device(w, dx, m, ddst, route=ROUTE_AUTO, stream=None):
    """Device-resident activations and result (DeviceBuffer or raw pointers)."""
    xp = dx.ptr if isinstance(dx, DeviceBuffer) else dx
    dp = ddst.ptr if isinstance(ddst, DeviceBuffer) else ddst
    check(lib.b200_mul_mat(w.ty, w.n_rows, w.k, m, w.ptr, xp, w.k, dp, w.n_rows, route, stream), "mul_mat")


def bench_mul_mat_q8(weights, act, act_kind, dst, m=1, reps=200):
    """event-timed microseconds per launch of b200_mul_mat_q8 over the given Weight copies, replayed as one CUDA graph"""
    arr = (C.c_void_p * len(weights))(*[w.ptr for w in weights])
    us = C.c_float(0)
    w = weights[0]
    check(lib.b200_bench_mul_mat_q8(w.ty, w.n_rows, w.k, m, arr, len(weights), act.ptr, act_kind, dst.ptr, reps, C.byref(us)), "bench_mul_mat_q8")
    return us.value


class Event:
    """A CUDA event on the library's launching stream."""

    def __init__(self):
        p = C.c_void_p()
        check(lib.b200_event_create(C.byref(p)), "event_create")
        self.ptr = p.value

    def record(self, stream=None):
        check(lib.b200_event_record(self.ptr, stream), "event_record")

    def synchronize(self):
        check(lib.b200_event_synchronize(self.ptr), "event_synchronize")

    def elapsed_ms(self, stop):
        ms = C.c_float()
        check(lib.b200_event_elapsed_ms(self.ptr, stop.ptr, C.byref(ms)), "event_elapsed")
        return ms.value

    def __del__(self):
        try:
            if self.ptr:
                lib.b200_event_destroy(self.ptr)
                self.ptr = None
        except Exception:
            pass


class ExpertWeights:
    """A quantized [n_expert, n, k] tensor on the device: one tile-layout matrix per expert, back to back."""

    def __init__(self, ty, blocks, n, k):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        self.ty, self.n, self.k = ty, int(n), int(k)
        row_bytes = self.k // 256 * GROUP_BYTES[ty]
        self.n_expert = blocks.size // (row_bytes * self.n)
        assert blocks.size == self.n_expert * self.n * row_bytes
        self.expert_bytes = lib.b200_weight_nbytes(ty, self.n, self.k)
        self.buf = DeviceBuffer(self.expert_bytes * self.n_expert)
        flat = blocks.reshape(self.n_expert, self.n * row_bytes)
        for e in range(self.n_expert):
            check(lib.b200_weight_upload(ty, self.n, self.k, flat[e].ctypes.data, self.buf.ptr + e * self.expert_bytes,
                                         None), "weight_upload")

    @property
    def ptr(self):
        return self.buf.ptr


def mul_mat_id(w, b, ids):
    """w: ExpertWeights; b: f32 [n_tok, ne11, k]; ids: i32 [n_tok, n_ids] -> f32 [n_tok, n_ids, n]."""
    b = np.ascontiguousarray(b, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    n_tok, ne11, k = b.shape
    n_ids = ids.shape[1]
    db, dids = device_array(b), device_array(ids)
    dst = DeviceBuffer(4 * n_tok * n_ids * w.n)
    check(lib.b200_mul_mat_id(w.ty, w.n, k, w.n_expert, ne11, n_tok, n_ids, w.ptr, db.ptr, dids.ptr, dst.ptr, 0, None),
          "mul_mat_id")
    return dst.download(np.float32, n_tok * n_ids * w.n).reshape(n_tok, n_ids, w.n)


class FlashAttnArgs(C.Structure):
    """struct b200_flash_attn_args"""
    _fields_ = [
        ("dk", C.c_int64), ("dv", C.c_int64), ("n_tok", C.c_int64), ("n_head", C.c_int64),
        ("n_head_kv", C.c_int64), ("n_kv", C.c_int64),
        ("q", C.c_void_p), ("q_nb1", C.c_int64), ("q_nb2", C.c_int64),
        ("k", C.c_void_p), ("k_nb1", C.c_int64), ("k_nb2", C.c_int64),
        ("v", C.c_void_p), ("v_nb1", C.c_int64), ("v_nb2", C.c_int64),
        ("mask", C.c_void_p), ("mask_nb1", C.c_int64),
        ("sinks", C.c_void_p),
        ("scale", C.c_float), ("max_bias", C.c_float), ("logit_softcap", C.c_float),
        ("dst", C.c_void_p),
        ("n_chunks", C.c_int32), ("mode", C.c_int32),
    ]


class KvCacheView:
    """K and V of one layer on the device, laid out like the reference's KV cache: position-major
    rows of [n_head_kv * d] f16 (crates/llama/src/kv_cache.rs:2528-2579)."""

    def __init__(self, k, v):
        """k: uint16 (f16 bits) [n_head_kv, n_kv, dk]; v: [n_head_kv, n_kv, dv] (head-major on the host)."""
        self.h_kv, self.n_kv, self.dk = k.shape
        self.dv = v.shape[2]
        kc = np.ascontiguousarray(np.transpose(k, (1, 0, 2)))  # [n_kv, h_kv, dk]
        vc = np.ascontiguousarray(np.transpose(v, (1, 0, 2)))
        self.k = device_array(kc)
        self.v = device_array(vc)
        self.k_nb1, self.k_nb2 = self.h_kv * self.dk * 2, self.dk * 2
        self.v_nb1, self.v_nb2 = self.h_kv * self.dv * 2, self.dv * 2


def flash_attn(q, kv, mask, scale, sinks=None, max_bias=0.0, softcap=0.0, n_chunks=0, mode=0, stream=None):
    """q: f32 [H, T, DK] host; kv: KvCacheView; mask: uint16 (f16 bits) [T, n_kv] or None -> f32 [T, H, DV]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    H, T, DK = q.shape
    dq = device_array(q)
    dst = DeviceBuffer(4 * T * H * kv.dv)
    a = FlashAttnArgs()
    a.dk, a.dv, a.n_tok, a.n_head, a.n_head_kv, a.n_kv = DK, kv.dv, T, H, kv.h_kv, kv.n_kv
    a.q, a.q_nb1, a.q_nb2 = dq.ptr, DK * 4, T * DK * 4
    a.k, a.k_nb1, a.k_nb2 = kv.k.ptr, kv.k_nb1, kv.k_nb2
    a.v, a.v_nb1, a.v_nb2 = kv.v.ptr, kv.v_nb1, kv.v_nb2
    keep = [dq, dst]
    if mask is not None:
        dm = device_array(np.ascontiguousarray(mask, dtype=np.uint16))
        keep.append(dm)
        a.mask, a.mask_nb1 = dm.ptr, kv.n_kv * 2
    else:
        a.mask, a.mask_nb1 = None, 0
    if sinks is not None:
        ds = device_array(np.ascontiguousarray(sinks, dtype=np.float32))
        keep.append(ds)
        a.sinks = ds.ptr
    else:
        a.sinks = None
    a.scale, a.max_bias, a.logit_softcap = scale, max_bias, softcap
    a.dst = dst.ptr
    a.n_chunks, a.mode = n_chunks, mode
    check(lib.b200_flash_attn_ext(C.byref(a), stream), "flash_attn_ext")
    return dst.download(np.float32, T * H * kv.dv).reshape(T, H, kv.dv)


def act_kind_for(ty, n=8, m=1):
    """The activation quantizer the reference's route for (type, n rows, m activation rows) reads."""
    if ty not in (Q4_K, Q6_K):
        return ACT_Q8_0
    if ty == Q4_K and n % 8 == 0 and m >= 4:
        return ACT_Q8_K_MIXED
    return ACT_Q8_K
