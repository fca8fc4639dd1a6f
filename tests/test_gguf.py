"""GGUF reader / writer (include/gguf_b200.h) on the CPU: the writer reproduces the reference writer's golden
file byte for byte (parity/gguf_write_ref.bin, cut into tests/golden/gguf_write_ref.bin), files round-trip,
and malformed files are refused with a status."""
import importlib
import os
import struct

import numpy as np
import pytest

import b200

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gguf_write_ref.bin")
F32, Q4_0, Q4_K = 0, 2, 12


@pytest.fixture(scope="module")
def gg():
    b200.load()
    return importlib.import_module("llama_rust_b200.gguf")


def lcg_bytes(n, state):
    out = []
    for _ in range(n):
        state[0] = (state[0] * 1664525 + 1013904223) & 0xFFFFFFFF
        out.append(state[0] >> 24)
    return np.array(out, dtype=np.uint8)


def reference_content(gg, path):
    """the logical content of crates/ggml/src/gguf_write.rs:239-266 (gguf_write_bit_exact_vs_reference)"""
    st = [0x12345678]
    a, b = lcg_bytes(64, st), lcg_bytes(18, st)
    w = gg.Writer(32)
    w.set("general.architecture", "test")
    w.set("test.block_count", 2)
    w.set("test.f", 1.5)
    w.set("test.arr", np.array([-1, 7, 42], dtype=np.int32))
    w.set("test.strs", ["alpha", "beta"])
    w.add_tensor("a.weight", F32, (16,), a)
    w.add_tensor("b.weight", Q4_0, (32,), b)
    w.write(path)
    return a, b


def test_writer_is_byte_identical_to_the_reference_writer(gg, tmp_path):
    p = tmp_path / "ref.gguf"
    reference_content(gg, p)
    assert p.read_bytes() == open(GOLDEN, "rb").read()


def test_reader_reads_the_reference_file(gg):
    r = gg.Reader(GOLDEN)
    assert r.version == 3 and r.str("general.architecture") == "test" and r.u32("test.block_count") == 2
    assert r.f32("test.f") == 1.5 and r.arr_len("test.arr") == 3 and r.arr_len("test.strs") == 2 and r.arr_len("test.f") == -1
    st = [0x12345678]
    a, b = lcg_bytes(64, st), lcg_bytes(18, st)
    (n0, t0, ne0, d0), (n1, t1, ne1, d1) = r.tensors()
    assert (n0, t0, ne0) == ("a.weight", F32, (16, 1, 1, 1)) and np.array_equal(d0, a)
    assert (n1, t1, ne1) == ("b.weight", Q4_0, (32, 1, 1, 1)) and np.array_equal(d1, b)
    assert r.data_offset % 32 == 0
    r.close()


def test_llama_file_round_trip(gg, tmp_path):
    ll = importlib.import_module("llama_rust_b200.llama")
    syn = importlib.import_module("llama_rust_b200.synth")
    hp = dict(n_vocab=512, n_embd=512, n_head=8, n_head_kv=2, n_embd_head=64, n_ff=1024, n_layer=2, n_ctx_train=4096, rope_mode=0,
              norm_rms_eps=1e-5, rope_freq_base=10000.0, rope_freq_scale=1.0)
    tensors = list(syn.llama_tensors(hp, lambda n: ll.q4_k_m_type(n, 2)))
    p = tmp_path / "tiny.gguf"
    gg.write_llama(p, hp, tensors)
    r = gg.Reader(p)
    assert r.str("general.architecture") == "llama" and r.u32("llama.block_count") == 2 and r.u32("llama.attention.head_count_kv") == 2
    assert abs(r.f32("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
    got = {n: (t, ne, d) for n, t, ne, d in r.tensors()}
    assert len(got) == len(tensors)
    for name, ty, arr, ne0, ne1 in tensors:
        t, ne, d = got[name]
        assert t == ty and ne[:2] == (ne0, ne1) and np.array_equal(d, np.ascontiguousarray(arr).view(np.uint8).ravel()), name
    r.close()


def test_malformed_files_are_refused(gg, tmp_path):
    m = b200.load()
    raw = open(GOLDEN, "rb").read()
    cases = {"magic": b"GGUX" + raw[4:], "version": raw[:4] + struct.pack("<I", 9) + raw[8:], "truncated": raw[:100],
             "short": raw[:10], "counts": raw[:8] + struct.pack("<Q", 1 << 60) + raw[16:]}
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(data)
        with pytest.raises(m.B200Error):
            gg.Reader(p)
    with pytest.raises(m.B200Error, match="cannot open"):
        gg.Reader(tmp_path / "missing.gguf")
    w = gg.Writer(32)
    with pytest.raises(m.B200Error, match="bytes given"):
        w.add_tensor("t", Q4_K, (256, 2), np.zeros(100, dtype=np.uint8))
    w.add_tensor("t", F32, (4,), np.zeros(4, dtype=np.float32))
    with pytest.raises(m.B200Error, match="duplicate"):
        w.add_tensor("t", F32, (4,), np.zeros(4, dtype=np.float32))


def crafted(kvs, tensors, alignment_pad=True, data=b""):
    """a GGUF v3 file written by hand: kvs = [(key, u32 value)], tensors = [(name, dims, type, offset)]"""
    out = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs)))
    for key, val in kvs:
        kb = key.encode()
        out += struct.pack("<Q", len(kb)) + kb + struct.pack("<II", 4, val)   # type 4 = u32
    for name, dims, ty, off in tensors:
        nb = name.encode()
        out += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d & 0xFFFFFFFFFFFFFFFF)
        out += struct.pack("<IQ", ty, off & 0xFFFFFFFFFFFFFFFF)
    if alignment_pad:
        out += b"\0" * (-len(out) % 32)
    return bytes(out) + data


def test_crafted_tensor_infos_are_refused(gg, tmp_path):
    """sizes and offsets from an untrusted file may not wrap around: a negative dimension, a byte count that
    overflows, an aligned offset near 2^64 whose sum with the data start wraps; empty and repeated keys
    (refused by the reference's reader too, crates/ggml/src/gguf.rs:509-512,554)"""
    m = b200.load()
    good = crafted([("a", 1)], [("t", (8,), F32, 0)], data=b"\0" * 32)
    p = tmp_path / "good.gguf"
    p.write_bytes(good)
    r = gg.Reader(p)
    assert [t[0] for t in r.tensors()] == ["t"]
    r.close()
    bad = {
        "negative dimension": crafted([], [("t", (-8,), F32, 0)], data=b"\0" * 32),
        "overflows": crafted([], [("t", (1 << 40, 1 << 40), F32, 0)], data=b"\0" * 32),
        "outside the file": crafted([], [("t", (8,), F32, 0xFFFFFFFFFFFFFFE0)], data=b"\0" * 32),
        "outside the file ": crafted([], [("t", (64,), F32, 0)], data=b"\0" * 32),
        "empty key": crafted([("", 1)], [], data=b""),
        "duplicate key": crafted([("a", 1), ("a", 2)], [], data=b""),
    }
    for why, blob in bad.items():
        p = tmp_path / "bad.gguf"
        p.write_bytes(blob)
        with pytest.raises(m.B200Error, match=why.strip()):
            gg.Reader(p)
