"""Pins the oracle's glue ops (rms_norm, silu, swiglu, add, rope, set_rows) to node outputs of the C
ggml build the reference ports, cut from its decode dump (tests/golden/glue_nodes.npz).  Bit-exact."""
import numpy as np
import pytest

import orc_glue
from conftest import bits_equal


@pytest.fixture(scope="module")
def nodes(golden):
    return golden("glue_nodes")


def cases(nodes, kind):
    return range(int(nodes[f"n_{kind}"]))


def test_rms_norm(nodes):
    assert int(nodes["n_rms_norm"]) >= 40
    for k in cases(nodes, "rms_norm"):
        assert bits_equal(orc_glue.rms_norm(nodes[f"rms_norm_{k}_x"], 1e-5), nodes[f"rms_norm_{k}_y"]), k


def test_silu_wide_and_tail(nodes):
    # rows of 8 run the libm tail only, rows of 32 run two 16-lane polynomial chunks: both are in the dump
    widths = set()
    for k in cases(nodes, "silu"):
        x = nodes[f"silu_{k}_x"]
        widths.add(x.shape[-1])
        assert bits_equal(orc_glue.silu(x, wide=True), nodes[f"silu_{k}_y"]), k
    assert any(w < 16 for w in widths) and any(w >= 16 for w in widths)


def test_swiglu(nodes):
    assert int(nodes["n_swiglu"]) > 0
    for k in cases(nodes, "swiglu"):
        y = orc_glue.swiglu(nodes[f"swiglu_{k}_x"], nodes[f"swiglu_{k}_g"], wide=True)
        assert bits_equal(y, nodes[f"swiglu_{k}_y"]), k
        # the op the Llama graph emits instead: silu then mul
        y2 = orc_glue.mul(orc_glue.silu(nodes[f"swiglu_{k}_x"], wide=True), nodes[f"swiglu_{k}_g"])
        assert bits_equal(y2, nodes[f"swiglu_{k}_y"]), k


def test_add(nodes):
    for k in cases(nodes, "add"):
        a, b = nodes[f"add_{k}_a"][None, :], nodes[f"add_{k}_b"][None, :]
        assert bits_equal(orc_glue.add(a, b)[0], nodes[f"add_{k}_y"]), k


def test_rope_neox_positions_0_to_13(nodes):
    seen = set()
    for k in cases(nodes, "rope"):
        pos = nodes[f"rope_{k}_pos"]
        seen.update(int(p) for p in pos)
        y = orc_glue.rope(nodes[f"rope_{k}_x"], pos, n_dims=16, mode=2, freq_base=10000.0, n_ctx_orig=512)
        assert bits_equal(y, nodes[f"rope_{k}_y"]), k
    assert seen == set(range(14))


def test_rope_normal_shares_cache_and_rotation(nodes):
    # mode 0 pairs channels (2i, 2i+1) with the same cache entry NEOX gives pair (i, i + n/2)
    x = nodes["rope_2_x"]
    pos = nodes["rope_2_pos"]
    neox = orc_glue.rope(x, pos, 16, 2, n_ctx_orig=512)
    perm = np.empty(16, dtype=np.int64)
    perm[0::2], perm[1::2] = np.arange(8), np.arange(8) + 8
    normal = orc_glue.rope(x[..., perm], pos, 16, 0, n_ctx_orig=512)
    assert bits_equal(normal, neox[..., perm])


def test_rope_partial_dims_copy_the_rest():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 2, 32)).astype(np.float32)
    y = orc_glue.rope(x, [5, 6, 7], n_dims=16, mode=0)
    assert bits_equal(y[..., 16:], x[..., 16:]) and not bits_equal(y[..., :16], x[..., :16])


def test_set_rows_f16(nodes):
    assert int(nodes["n_set_rows"]) >= 4
    for k in cases(nodes, "set_rows"):
        x, idx, want = nodes[f"set_rows_{k}_x"], nodes[f"set_rows_{k}_idx"], nodes[f"set_rows_{k}_y"]
        dst = np.zeros((512, x.shape[1]), dtype=np.uint16)
        orc_glue.set_rows_f16(x, idx, dst)
        assert np.array_equal(dst[idx], want.view(np.uint16)), k
        untouched = np.setdiff1d(np.arange(512), idx)
        assert not dst[untouched].any()


def test_argmax_ties_take_the_last():
    assert orc_glue.argmax(np.array([1, 5, 2, 5, 0], dtype=np.float32)) == 3
    assert orc_glue.argmax(np.array([-np.inf, -np.inf], dtype=np.float32)) == 1


def test_get_rows_dequantizes():
    import orc
    rng = np.random.default_rng(5)
    w = rng.standard_normal((40, 256)).astype(np.float32)
    q = orc.quantize_rows(orc.Q4_K, w)
    rows = orc_glue.get_rows(orc.Q4_K, q, 256, 40, [7, 0, 39])
    full = orc.dequantize(orc.Q4_K, q, 256)
    assert bits_equal(rows, full[[7, 0, 39]])
