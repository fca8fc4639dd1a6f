"""The FLASH_ATTN_EXT oracle against the reference's golden dumps (bit-exact).

tests/golden/flash_attn.npz holds the 13 F16-KV cases of parity/fa_ref.bin (tiled and
one_chunk paths, sinks, softcap, ALiBi, DV != DK, GQA decode), flash_attn_probe.npz the
S_kv = 600 probes of parity/fa_probe.bin whose 1-row runs take the split-KV path with
1 and 8 chunks (crates/ggml/src/flash_attn.rs:2147,2195,2541 replay the same files).
"""
import numpy as np
import pytest

import orc
from conftest import bits_equal


def load_case(g, c):
    mode, dk, dv, h, hkv, t, skv, kty, vty = (int(v) for v in g[c + "/hdr"])
    q = g[c + "/q"].reshape(h, t, dk)
    k = g[c + "/k"].reshape(hkv, skv, dk)
    v = g[c + "/v"].reshape(hkv, skv, dv)
    mask = g[c + "/mask"].reshape(t, skv) if g[c + "/mask"].size else None
    sinks = g[c + "/sinks"] if g[c + "/sinks"].size else None
    scale, max_bias, softcap, _ = (float(x) for x in g[c + "/params"])
    return dict(q=q, k=k, v=v, mask=mask, sinks=sinks, scale=scale, max_bias=max_bias, softcap=softcap,
                dst=g[c + "/dst"].reshape(t, h, dv), T=t)


def case_names(g):
    return sorted({k.split("/")[0] for k in g.files if k.startswith("case")}, key=lambda s: int(s[4:]))


def test_reference_dump_cases_bit_exact(golden):
    g = golden("flash_attn")
    names = case_names(g)
    assert len(names) == 13
    paths = set()
    for c in names:
        d = load_case(g, c)
        out, path = orc.flash_attn(d["q"], d["k"], d["v"], d["mask"], d["scale"], sinks=d["sinks"],
                                   max_bias=d["max_bias"], softcap=d["softcap"])
        assert path == (orc.FA_TILED if d["T"] >= 64 else orc.FA_ONE_CHUNK)
        assert bits_equal(out, d["dst"]), c
        paths.add(path)
    assert paths == {orc.FA_TILED, orc.FA_ONE_CHUNK}


def test_split_kv_probe_bit_exact(golden):
    g = golden("flash_attn_probe")
    probes = sorted({k.split("/")[0] for k in g.files})
    checked = 0
    for p in probes:
        dk, dv, h, hkv, t, skv = (int(x) for x in g[p + "/geom"])
        scale, max_bias, softcap = (float(x) for x in g[p + "/knobs"])
        q = g[p + "/q"].reshape(h, t, dk)
        k = g[p + "/k"].reshape(hkv, skv, dk)
        v = g[p + "/v"].reshape(hkv, skv, dv)
        mask = g[p + "/mask"].reshape(t, skv)
        for r in sorted(x for x in g.files if x.startswith(p + "/rec/")):
            tag, tt, nth = (int(x) for x in r.split("/")[2:])
            if tag == 0:
                out, path = orc.flash_attn(q, k, v, mask, scale, n_chunks=nth)
                assert path == (orc.FA_SPLIT_KV if t == 1 else orc.FA_ONE_CHUNK)
            elif tag == 1:
                out, path = orc.flash_attn(q[:, tt:tt + 1], k, v, mask[tt:tt + 1], scale, n_chunks=nth)
                assert path == orc.FA_SPLIT_KV
            else:
                out, path = orc.flash_attn(q[:, 1:], k, v, mask[1:], scale)
            assert bits_equal(out.ravel(), g[r]), r
            checked += 1
    assert checked == 16


def test_split_kv_with_one_chunk_equals_one_chunk():
    """A single chunk merges exactly (crates/ggml/src/flash_attn.rs:1367-1370)."""
    rng = np.random.default_rng(0)
    H, Hkv, D, n_kv = 8, 2, 64, 700
    q = rng.standard_normal((H, 1, D)).astype(np.float32)
    k = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    v = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    a, _ = orc.flash_attn(q, k, v, None, 0.125, mode=orc.FA_SPLIT_KV, n_chunks=1)
    b, _ = orc.flash_attn(q, k, v, None, 0.125, mode=orc.FA_ONE_CHUNK)
    assert bits_equal(a, b)
