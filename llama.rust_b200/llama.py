"""ctypes wrapper of the Llama decode driver (include/llama_b200.h): weights in, tokens in, logits out.
Everything runs in libggml-b200.so; this module only moves host arrays across the C ABI."""
import ctypes as C

import numpy as np

from . import F32, check, lib

vp, i32, i64, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t


class HParams(C.Structure):
    _fields_ = [("n_vocab", i32), ("n_embd", i32), ("n_head", i32), ("n_head_kv", i32), ("n_embd_head", i32), ("n_ff", i32),
                ("n_layer", i32), ("n_ctx_train", i32), ("rope_mode", i32), ("norm_rms_eps", C.c_float),
                ("rope_freq_base", C.c_float), ("rope_freq_scale", C.c_float)]


lib.b200_llama_new.argtypes = [C.POINTER(HParams), i32, i32, i32, i32, C.POINTER(vp)]
lib.b200_llama_free.argtypes = [vp]
lib.b200_llama_free.restype = None
lib.b200_llama_set_tensor.argtypes = [vp, C.c_char_p, i32, i64, i64, vp, sz]
lib.b200_llama_set_tensor_shard.argtypes = [vp, C.c_char_p, i32, i64, i64, vp, sz]
lib.b200_llama_decode.argtypes = [vp, vp, vp, i32, vp, vp]
lib.b200_llama_decode_seqs.argtypes = [vp, vp, vp, vp, i32, vp, i32, vp, vp]
lib.b200_llama_kv_clear.argtypes = [vp]
lib.b200_llama_kv_used.argtypes = [vp]
lib.b200_llama_kv_used.restype = i32
lib.b200_llama_replay.argtypes = [vp, i32, C.POINTER(C.c_float)]
lib.b200_llama_read_node.argtypes = [vp, C.c_char_p, vp, sz]
lib.b200_llama_new_tp.argtypes = [C.POINTER(HParams), i32, i32, i32, i32, i32, i32, vp, C.POINTER(vp)]
TP_HOOK = C.CFUNCTYPE(C.c_int, vp, C.c_int, C.c_int, C.c_int, vp, i64, vp, i64, i64)
lib.b200_llama_new_tp_hook.argtypes = [C.POINTER(HParams), i32, i32, i32, i32, i32, i32, TP_HOOK, vp, C.POINTER(vp)]
lib.b200_llama_tp_exchange_kind.argtypes = [vp]
lib.b200_tp_unique_id.argtypes = [vp]
lib.b200_tp_shard_shape.argtypes = [C.c_char_p, i32, i64, i64, i32, C.POINTER(i32), C.POINTER(i64), C.POINTER(i64)]
lib.b200_tp_shard_tensor.argtypes = [C.c_char_p, i32, i64, i64, vp, i32, i32, vp, sz]

from .shapes import LLAMA3_8B, LLAMA3_70B, q4_k_m_type, tensor_shapes, use_more_bits  # noqa: E402,F401  (pure Python: importable without the library)


def tp_unique_id():
    """128 bytes (an ncclUniqueId) made on one rank, to be handed to every rank of a tensor-parallel group"""
    buf = (C.c_uint8 * 128)()
    check(lib.b200_tp_unique_id(buf), "tp_unique_id")
    return bytes(buf)


def tp_shard_shape(name, ty, ne0, ne1, tp_size):
    """-> (split, ne0_local, ne1_local); split: 0 replicated, 1 rows, 2 K"""
    split, l0, l1 = i32(0), i64(0), i64(0)
    check(lib.b200_tp_shard_shape(name.encode(), ty, ne0, ne1, tp_size, C.byref(split), C.byref(l0), C.byref(l1)), f"tp_shard_shape {name}")
    return split.value, l0.value, l1.value


def tp_shard_tensor(name, ty, blocks, ne0, ne1, tp_rank, tp_size):
    """this rank's shard of a whole tensor, as a uint8 array"""
    blocks = np.ascontiguousarray(blocks)
    _, l0, l1 = tp_shard_shape(name, ty, ne0, ne1, tp_size)
    out = np.empty(blocks.nbytes * (l0 * l1) // (ne0 * ne1), dtype=np.uint8)
    check(lib.b200_tp_shard_tensor(name.encode(), ty, ne0, ne1, blocks.ctypes.data, tp_rank, tp_size, out.ctypes.data, out.nbytes),
          f"tp_shard_tensor {name}")
    return out


class Llama:
    def __init__(self, hp, n_ctx, n_batch, device=0, cpu_threads=8, tp_rank=0, tp_size=1, tp_id=None, tp_hook=None):
        """tp_hook(kind, rank, size, dev_buf, count, dev_dst, n_local, rows) -> 0: a tensor-parallel rank whose
        collectives the host carries out (b200_llama_new_tp_hook), for tests that play several ranks on one GPU"""
        self.hp = dict(hp)
        h = HParams(**self.hp)
        p = vp()
        if tp_size > 1 and tp_hook is not None:
            self._hook = TP_HOOK(lambda user, kind, rank, size, buf, count, dst, n_local, rows:
                                 int(tp_hook(kind, rank, size, buf, count, dst, n_local, rows)))
            check(lib.b200_llama_new_tp_hook(C.byref(h), device, n_ctx, n_batch, cpu_threads, tp_rank, tp_size, self._hook, None, C.byref(p)),
                  "llama_new_tp_hook")
        elif tp_size > 1:
            idbuf = (C.c_uint8 * 128).from_buffer_copy(tp_id)
            check(lib.b200_llama_new_tp(C.byref(h), device, n_ctx, n_batch, cpu_threads, tp_rank, tp_size, idbuf, C.byref(p)), "llama_new_tp")
        else:
            check(lib.b200_llama_new(C.byref(h), device, n_ctx, n_batch, cpu_threads, C.byref(p)), "llama_new")
        self.ptr = p.value

    def set_tensor(self, name, ty, blocks, ne0, ne1):
        blocks = np.ascontiguousarray(blocks)
        check(lib.b200_llama_set_tensor(self.ptr, name.encode(), ty, ne0, ne1, blocks.ctypes.data, blocks.nbytes), f"set_tensor {name}")

    def set_tensor_shard(self, name, ty, blocks, ne0_local, ne1_local):
        """a tensor-parallel rank's own shard, already cut (tp_shard_shape gives the local shape)"""
        blocks = np.ascontiguousarray(blocks)
        check(lib.b200_llama_set_tensor_shard(self.ptr, name.encode(), ty, ne0_local, ne1_local, blocks.ctypes.data, blocks.nbytes),
              f"set_tensor_shard {name}")

    def decode(self, tokens, pos, logits=True, argmax=False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        out = np.empty(self.hp["n_vocab"], dtype=np.float32) if logits else None
        am = C.c_int32(-1)
        check(lib.b200_llama_decode(self.ptr, tokens.ctypes.data, pos.ctypes.data, tokens.size,
                                    out.ctypes.data if logits else None, C.byref(am) if argmax else None), "llama_decode")
        if logits and argmax:
            return out, am.value
        return out if logits else (am.value if argmax else None)

    def decode_seqs(self, tokens, pos, seq_ids, out_rows, logits=True, argmax=False):
        """several sequences in one step -> (logits [n_out, n_vocab] or None, argmax [n_out] or None)"""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        seq_ids = np.ascontiguousarray(seq_ids, dtype=np.int32)
        out_rows = np.ascontiguousarray(out_rows, dtype=np.int32)
        out = np.empty((out_rows.size, self.hp["n_vocab"]), dtype=np.float32) if logits else None
        am = np.empty(out_rows.size, dtype=np.int32) if argmax else None
        check(lib.b200_llama_decode_seqs(self.ptr, tokens.ctypes.data, pos.ctypes.data, seq_ids.ctypes.data, tokens.size,
                                         out_rows.ctypes.data, out_rows.size, out.ctypes.data if logits else None,
                                         am.ctypes.data if argmax else None), "llama_decode_seqs")
        return out, am

    def tp_exchange_kind(self):
        """1: the library's single-kernel exchange over peer memory, 0: NCCL, -1: not tensor parallel (or a hook)"""
        return lib.b200_llama_tp_exchange_kind(self.ptr)

    def kv_clear(self):
        check(lib.b200_llama_kv_clear(self.ptr), "kv_clear")

    def kv_used(self):
        return lib.b200_llama_kv_used(self.ptr)

    def read_node(self, name, count, dtype=np.float32):
        """the last decode call's tensor of that name (b200_llama_read_node), `count` elements"""
        out = np.empty(count, dtype=dtype)
        check(lib.b200_llama_read_node(self.ptr, name.encode(), out.ctypes.data, out.nbytes), f"read_node {name}")
        return out

    def replay(self, reps):
        ms = C.c_float(0)
        check(lib.b200_llama_replay(self.ptr, reps, C.byref(ms)), "llama_replay")
        return ms.value

    def close(self):
        if self.ptr:
            lib.b200_llama_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
