"""ctypes wrapper of the GGUF reader / writer and the GGUF loader of the decode driver (include/gguf_b200.h,
include/llama_b200.h)."""
import ctypes as C

import numpy as np

from . import check, lib
from .llama import HParams, Llama

vp, i32, i64, u32, u64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_size_t
lib.b200_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
lib.b200_gguf_close.argtypes = [vp]
lib.b200_gguf_close.restype = None
lib.b200_gguf_version.argtypes = [vp]
lib.b200_gguf_version.restype = u32
lib.b200_gguf_n_kv.argtypes = [vp]
lib.b200_gguf_n_kv.restype = i64
lib.b200_gguf_n_tensors.argtypes = [vp]
lib.b200_gguf_n_tensors.restype = i64
lib.b200_gguf_data_offset.argtypes = [vp]
lib.b200_gguf_data_offset.restype = u64
lib.b200_gguf_tensor.argtypes = [vp, i64, C.POINTER(C.c_char_p), C.POINTER(i32), C.POINTER(i64 * 4), C.POINTER(vp), C.POINTER(sz)]
lib.b200_gguf_find_tensor.argtypes = [vp, C.c_char_p]
lib.b200_gguf_get_u32.argtypes = [vp, C.c_char_p, C.POINTER(u32)]
lib.b200_gguf_get_f32.argtypes = [vp, C.c_char_p, C.POINTER(C.c_float)]
lib.b200_gguf_get_str.argtypes = [vp, C.c_char_p, C.c_char_p, sz]
lib.b200_gguf_arr_len.argtypes = [vp, C.c_char_p]
lib.b200_gguf_arr_len.restype = i64
lib.b200_gguf_writer_new.argtypes = [u64, C.POINTER(vp)]
lib.b200_gguf_writer_free.argtypes = [vp]
lib.b200_gguf_writer_free.restype = None
lib.b200_gguf_set_u32.argtypes = [vp, C.c_char_p, u32]
lib.b200_gguf_set_f32.argtypes = [vp, C.c_char_p, C.c_float]
lib.b200_gguf_set_str.argtypes = [vp, C.c_char_p, C.c_char_p]
lib.b200_gguf_set_arr.argtypes = [vp, C.c_char_p, u32, vp, u64]
lib.b200_gguf_set_arr_str.argtypes = [vp, C.c_char_p, C.POINTER(C.c_char_p), u64]
lib.b200_gguf_add_tensor.argtypes = [vp, C.c_char_p, i32, C.POINTER(i64 * 4), vp, sz]
lib.b200_gguf_write.argtypes = [vp, C.c_char_p]
lib.b200_llama_load_gguf.argtypes = [C.c_char_p, i32, i32, i32, i32, C.POINTER(vp)]
lib.b200_llama_get_hparams.argtypes = [vp, C.POINTER(HParams)]


class Reader:
    def __init__(self, path):
        p = vp()
        check(lib.b200_gguf_open(str(path).encode(), C.byref(p)), "gguf_open")
        self.ptr = p.value

    def close(self):
        if self.ptr:
            lib.b200_gguf_close(self.ptr)
            self.ptr = None

    @property
    def version(self):
        return lib.b200_gguf_version(self.ptr)

    @property
    def data_offset(self):
        return lib.b200_gguf_data_offset(self.ptr)

    def u32(self, key):
        v = u32(0)
        check(lib.b200_gguf_get_u32(self.ptr, key.encode(), C.byref(v)), key)
        return v.value

    def f32(self, key):
        v = C.c_float(0)
        check(lib.b200_gguf_get_f32(self.ptr, key.encode(), C.byref(v)), key)
        return v.value

    def str(self, key):
        buf = C.create_string_buffer(4096)
        check(lib.b200_gguf_get_str(self.ptr, key.encode(), buf, 4096), key)
        return buf.value.decode()

    def arr_len(self, key):
        return lib.b200_gguf_arr_len(self.ptr, key.encode())

    def tensors(self):
        """[(name, type, ne tuple, bytes as uint8 array copied out of the map)]"""
        out = []
        for i in range(lib.b200_gguf_n_tensors(self.ptr)):
            name, ty, ne, data, n = C.c_char_p(), i32(0), (i64 * 4)(), vp(), sz(0)
            check(lib.b200_gguf_tensor(self.ptr, i, C.byref(name), C.byref(ty), C.byref(ne), C.byref(data), C.byref(n)), "gguf_tensor")
            raw = np.ctypeslib.as_array(C.cast(data, C.POINTER(C.c_uint8)), shape=(n.value,)).copy() if n.value else np.empty(0, np.uint8)
            out.append((name.value.decode(), ty.value, tuple(ne), raw))
        return out


class Writer:
    def __init__(self, alignment=32):
        p = vp()
        check(lib.b200_gguf_writer_new(alignment, C.byref(p)), "gguf_writer_new")
        self.ptr, self.keep = p.value, []

    def set(self, key, value):
        k = key.encode()
        if isinstance(value, str):
            check(lib.b200_gguf_set_str(self.ptr, k, value.encode()), key)
        elif isinstance(value, float):
            check(lib.b200_gguf_set_f32(self.ptr, k, value), key)
        elif isinstance(value, int):
            check(lib.b200_gguf_set_u32(self.ptr, k, value), key)
        elif isinstance(value, (list, tuple)) and value and isinstance(value[0], str):
            arr = (C.c_char_p * len(value))(*[v.encode() for v in value])
            check(lib.b200_gguf_set_arr_str(self.ptr, k, arr, len(value)), key)
        else:
            a = np.ascontiguousarray(value)
            ids = {np.dtype(np.int32): 5, np.dtype(np.uint32): 4, np.dtype(np.float32): 6, np.dtype(np.uint8): 0, np.dtype(np.int64): 11}
            check(lib.b200_gguf_set_arr(self.ptr, k, ids[a.dtype], a.ctypes.data, a.size), key)

    def add_tensor(self, name, ty, ne, data):
        data = np.ascontiguousarray(data)
        self.keep.append(data)
        ne4 = (i64 * 4)(*(list(ne) + [1] * (4 - len(ne))))
        check(lib.b200_gguf_add_tensor(self.ptr, name.encode(), ty, C.byref(ne4), data.ctypes.data, data.nbytes), name)

    def write(self, path):
        check(lib.b200_gguf_write(self.ptr, str(path).encode()), "gguf_write")

    def __del__(self):
        if getattr(self, "ptr", None):
            lib.b200_gguf_writer_free(self.ptr)
            self.ptr = None


def write_llama(path, hp, tensors, name="synthetic"):
    """tensors: iterable of (gguf name, type, array, ne0, ne1).  The llama.* keys the reference's loader reads
    (crates/llama/src/model.rs) plus a placeholder tokenizer-free header."""
    w = Writer(32)
    w.set("general.architecture", "llama")
    w.set("general.name", name)
    w.set("llama.block_count", hp["n_layer"])
    w.set("llama.context_length", hp["n_ctx_train"])
    w.set("llama.embedding_length", hp["n_embd"])
    w.set("llama.feed_forward_length", hp["n_ff"])
    w.set("llama.attention.head_count", hp["n_head"])
    w.set("llama.attention.head_count_kv", hp["n_head_kv"])
    w.set("llama.attention.key_length", hp["n_embd_head"])
    w.set("llama.attention.value_length", hp["n_embd_head"])
    w.set("llama.rope.dimension_count", hp["n_embd_head"])
    w.set("llama.attention.layer_norm_rms_epsilon", float(hp["norm_rms_eps"]))
    w.set("llama.rope.freq_base", float(hp["rope_freq_base"]))
    w.set("llama.vocab_size", hp["n_vocab"])
    for tname, ty, arr, ne0, ne1 in tensors:
        w.add_tensor(tname, ty, (ne0, ne1), arr)
    w.write(path)


def load_llama(path, n_ctx, n_batch, device=0, cpu_threads=8):
    """-> Llama (include/llama_b200.h b200_llama_load_gguf)"""
    p = vp()
    check(lib.b200_llama_load_gguf(str(path).encode(), device, n_ctx, n_batch, cpu_threads, C.byref(p)), "llama_load_gguf")
    h = HParams()
    check(lib.b200_llama_get_hparams(p.value, C.byref(h)), "llama_get_hparams")
    obj = Llama.__new__(Llama)
    obj.hp = {f: getattr(h, f) for f, _ in HParams._fields_}
    obj.ptr = p.value
    return obj
