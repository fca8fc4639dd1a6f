"""ctypes binding of the oracle's glue ops and Llama forward (oracle/oracle_glue.cpp).
Test infrastructure, like tests/orc.py."""
import ctypes as C

import numpy as np

import orc

_ready = False
vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int32, C.c_float


def L():
    global _ready
    lib = orc.lib()
    if not _ready:
        lib.orc_rms_norm.argtypes = [vp, vp, i64, i64, f32]
        lib.orc_add.argtypes = [vp, vp, vp, i64, i64, i64, i64]
        lib.orc_mul.argtypes = [vp, vp, vp, i64, i64, i64, i64]
        lib.orc_silu.argtypes = [vp, vp, i64, i64, i32]
        lib.orc_swiglu.argtypes = [vp, vp, vp, i64, i64, i32]
        lib.orc_rope_cache.argtypes = [i32, i64, vp, i32, i32, f32, f32, f32, f32, f32, f32, vp]
        lib.orc_rope.argtypes = [vp, vp, i64, i64, i64, vp, vp, i32, i32, i32, f32, f32, f32, f32, f32, f32]
        lib.orc_set_rows_f16.argtypes = [vp, i64, i64, vp, vp, i64]
        lib.orc_get_rows.argtypes = [i32, vp, i64, i64, vp, i64, vp]
        lib.orc_argmax.argtypes = [vp, i64]
        lib.orc_argmax.restype = i32
        lib.orc_llama_forward.argtypes = [vp, vp, vp, i64, i64, vp, vp, vp, i64, vp, i32, i32, i32]
        lib.orc_llama_forward_tp.argtypes = [vp, vp, vp, i64, i64, vp, vp, vp, i64, vp, i32, i32, i32, vp, vp]
        _ready = True
    return lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def rms_norm(x, eps):
    x = _f(x)
    y = np.empty_like(x)
    L().orc_rms_norm(x.ctypes.data, y.ctypes.data, x.shape[-1], x.size // x.shape[-1], eps)
    return y


def _bin(fn, a, b):
    a, b = _f(a), _f(b)
    y = np.empty_like(a)
    ne0 = a.shape[-1]
    fn(a.ctypes.data, b.ctypes.data, y.ctypes.data, ne0, a.size // ne0, b.shape[-1], b.size // b.shape[-1])
    return y


def add(a, b):
    return _bin(L().orc_add, a, b)


def mul(a, b):
    return _bin(L().orc_mul, a, b)


def silu(x, wide=True):
    x = _f(x)
    y = np.empty_like(x)
    L().orc_silu(x.ctypes.data, y.ctypes.data, x.shape[-1], x.size // x.shape[-1], int(wide))
    return y


def swiglu(x, g, wide=True):
    x, g = _f(x), _f(g)
    y = np.empty_like(x)
    L().orc_swiglu(x.ctypes.data, g.ctypes.data, y.ctypes.data, x.shape[-1], x.size // x.shape[-1], int(wide))
    return y


def rope(x, pos, n_dims, mode, freq_base=10000.0, freq_scale=1.0, n_ctx_orig=4096, ext_factor=0.0, attn_factor=1.0,
         beta_fast=32.0, beta_slow=1.0, freq_factors=None):
    """x: [n_tok, n_head, ne0]"""
    x = _f(x)
    pos = np.ascontiguousarray(pos, dtype=np.int32)
    y = np.empty_like(x)
    ff = None if freq_factors is None else _f(freq_factors)
    rc = L().orc_rope(x.ctypes.data, y.ctypes.data, x.shape[2], x.shape[1], x.shape[0], pos.ctypes.data,
                      None if ff is None else ff.ctypes.data, n_dims, mode, n_ctx_orig, freq_base, freq_scale, ext_factor,
                      attn_factor, beta_fast, beta_slow)
    assert rc == 0
    return y


def rope_cache(pos, ne0, n_dims, freq_base=10000.0, freq_scale=1.0, n_ctx_orig=4096, ext_factor=0.0, attn_factor=1.0,
               beta_fast=32.0, beta_slow=1.0):
    c = np.empty(ne0, dtype=np.float32)
    L().orc_rope_cache(int(pos), ne0, None, n_dims, n_ctx_orig, freq_base, freq_scale, ext_factor, attn_factor, beta_fast,
                       beta_slow, c.ctypes.data)
    return c


def set_rows_f16(x, idx, dst):
    """writes rows of f32 x into the uint16 (f16 bits) array dst [rows, ne0] in place"""
    x = _f(x)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    assert dst.dtype == np.uint16 and dst.flags.c_contiguous
    rc = L().orc_set_rows_f16(x.ctypes.data, x.shape[-1], x.size // x.shape[-1], idx.ctypes.data, dst.ctypes.data, dst.shape[0])
    assert rc == 0
    return dst


def get_rows(ty, table, ne0, table_rows, ids):
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    y = np.empty((ids.size, ne0), dtype=np.float32)
    rc = L().orc_get_rows(ty, table.ctypes.data, ne0, table_rows, ids.ctypes.data, ids.size, y.ctypes.data)
    assert rc == 0
    return y


def argmax(x):
    x = _f(x)
    return int(L().orc_argmax(x.ctypes.data, x.size))


class LlamaLayer(C.Structure):
    _fields_ = [(n, vp) for n in ("wq", "wk", "wv", "wo", "gate", "up", "down")] + \
               [(n, i32) for n in ("tq", "tk", "tv", "to", "tg", "tu", "td")] + \
               [("attn_norm", vp), ("ffn_norm", vp), ("k_cache", vp), ("v_cache", vp)]


class LlamaModel(C.Structure):
    _fields_ = [(n, i32) for n in ("n_vocab", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_layer", "rope_mode",
                                   "n_ctx_orig", "tok_type", "out_type")] + \
               [("norm_eps", f32), ("freq_base", f32), ("freq_scale", f32), ("tok_embd", vp), ("out_norm", vp),
                ("output", vp), ("layers", C.POINTER(LlamaLayer)), ("kv_size", i64)]


class Llama:
    """The oracle's Llama: weights given as {gguf tensor name: (type, ndarray of ggml blocks or f32)}."""

    def __init__(self, hp, tensors, kv_size):
        self.hp, self.tensors, self.kv_size = hp, tensors, kv_size
        nl = hp["n_layer"]
        ek = hp["n_head_kv"] * hp["head_dim"]
        self.k = [np.zeros((kv_size, ek), dtype=np.uint16) for _ in range(nl)]
        self.v = [np.zeros((kv_size, ek), dtype=np.uint16) for _ in range(nl)]
        self.layers = (LlamaLayer * nl)()
        for il in range(nl):
            ly = self.layers[il]
            for field, tname, tfield in (("wq", "attn_q", "tq"), ("wk", "attn_k", "tk"), ("wv", "attn_v", "tv"),
                                         ("wo", "attn_output", "to"), ("gate", "ffn_gate", "tg"), ("up", "ffn_up", "tu"),
                                         ("down", "ffn_down", "td")):
                ty, arr = tensors[f"blk.{il}.{tname}.weight"]
                setattr(ly, field, arr.ctypes.data)
                setattr(ly, tfield, ty)
            ly.attn_norm = tensors[f"blk.{il}.attn_norm.weight"][1].ctypes.data
            ly.ffn_norm = tensors[f"blk.{il}.ffn_norm.weight"][1].ctypes.data
            ly.k_cache, ly.v_cache = self.k[il].ctypes.data, self.v[il].ctypes.data
        m = LlamaModel()
        for n in ("n_vocab", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_layer", "rope_mode", "n_ctx_orig"):
            setattr(m, n, hp[n])
        m.norm_eps, m.freq_base, m.freq_scale = hp["norm_eps"], hp["freq_base"], hp["freq_scale"]
        m.tok_type, tok = tensors["token_embd.weight"]
        m.tok_embd = tok.ctypes.data
        m.out_type, outw = tensors["output.weight"]
        m.output = outw.ctypes.data
        m.out_norm = tensors["output_norm.weight"][1].ctypes.data
        m.layers = self.layers
        m.kv_size = kv_size
        self.m = m

    def forward(self, tokens, pos, n_kv, mask, row_idx, out_ids, n_threads=8, wide_silu=True, keep_repacked=False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        mask = np.ascontiguousarray(mask, dtype=np.uint16)
        row_idx = np.ascontiguousarray(row_idx, dtype=np.int64)
        out_ids = np.ascontiguousarray(out_ids, dtype=np.int32)
        logits = np.empty((out_ids.size, self.hp["n_vocab"]), dtype=np.float32)
        rc = L().orc_llama_forward(C.byref(self.m), tokens.ctypes.data, pos.ctypes.data, tokens.size, n_kv, mask.ctypes.data,
                                   row_idx.ctypes.data, out_ids.ctypes.data, out_ids.size, logits.ctypes.data, n_threads,
                                   int(wide_silu), int(keep_repacked))
        assert rc == 0, f"orc_llama_forward failed ({rc})"
        return logits

    def forward_tp(self, tokens, pos, n_kv, mask, row_idx, out_ids, tp, n_threads=8, wide_silu=True, partials=False):
        """The forward pass as tp tensor-parallel ranks compute it: attn_output and ffn_down cut along K, the
        partial results added in rank order.  With partials=True also returns layer 0's per-rank partial results
        of attn_output and ffn_down, each [tp, n_tok, n_embd]."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        pos = np.ascontiguousarray(pos, dtype=np.int32)
        mask = np.ascontiguousarray(mask, dtype=np.uint16)
        row_idx = np.ascontiguousarray(row_idx, dtype=np.int64)
        out_ids = np.ascontiguousarray(out_ids, dtype=np.int32)
        logits = np.empty((out_ids.size, self.hp["n_vocab"]), dtype=np.float32)
        pa = np.zeros((tp, tokens.size, self.hp["n_embd"]), dtype=np.float32) if partials else None
        pf = np.zeros((tp, tokens.size, self.hp["n_embd"]), dtype=np.float32) if partials else None
        rc = L().orc_llama_forward_tp(C.byref(self.m), tokens.ctypes.data, pos.ctypes.data, tokens.size, n_kv, mask.ctypes.data,
                                      row_idx.ctypes.data, out_ids.ctypes.data, out_ids.size, logits.ctypes.data, n_threads,
                                      int(wide_silu), tp, pa.ctypes.data if partials else None, pf.ctypes.data if partials else None)
        assert rc == 0, f"orc_llama_forward_tp failed ({rc})"
        return (logits, pa, pf) if partials else logits
