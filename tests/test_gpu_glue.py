"""The glue-op kernels (RMS_NORM, ADD/MUL, SILU, ROPE, SET_ROWS, GET_ROWS, ARGMAX) through the C ABI,
against the reference's node dump (tests/golden/glue_nodes.npz) and against the CPU oracle on seeded
inputs of decoder sizes.  Bit-exact throughout."""
import importlib

import numpy as np
import pytest

import b200
import orc
import orc_glue
from conftest import bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    b200.load()
    return importlib.import_module("llama_rust_b200.glue")


@pytest.fixture(scope="module")
def nodes(golden):
    return golden("glue_nodes")


def activations(rng, shape, scale=1.0):
    # wide dynamic range like a residual stream: mostly unit scale, a few large channels
    x = rng.standard_normal(shape).astype(np.float32) * scale
    x[..., ::97] *= 30.0
    return x


def test_rms_norm_reference_dump(g, nodes):
    for k in range(int(nodes["n_rms_norm"])):
        assert bits_equal(g.rms_norm(nodes[f"rms_norm_{k}_x"], 1e-5), nodes[f"rms_norm_{k}_y"]), k


@pytest.mark.parametrize("ne0,rows", [(4096, 1), (4096, 16), (4096, 512), (8192, 3), (256, 7), (5120, 33), (100, 5)])
def test_rms_norm_and_weight(g, ne0, rows):
    rng = np.random.default_rng(ne0 + rows)
    x = activations(rng, (rows, ne0))
    w = (1.0 + 0.1 * rng.standard_normal(ne0)).astype(np.float32)
    y, yw = g.rms_norm(x, 1e-5, weight=w)
    want = orc_glue.rms_norm(x, 1e-5)
    assert bits_equal(y, want)
    assert bits_equal(yw, orc_glue.mul(want, w[None, :]))
    assert bits_equal(g.rms_norm(x, 1e-6), orc_glue.rms_norm(x, 1e-6))


def test_add_reference_dump(g, nodes):
    for k in range(int(nodes["n_add"])):
        a, b = nodes[f"add_{k}_a"][None, :], nodes[f"add_{k}_b"][None, :]
        assert bits_equal(g.add(a, b)[0], nodes[f"add_{k}_y"]), k


@pytest.mark.parametrize("shape,bshape", [((16, 4096), (16, 4096)), ((16, 4096), (1, 4096)), ((512, 14336), (512, 14336)),
                                          ((5, 64), (1, 1)), ((3, 64), (1, 16))])
def test_add_mul_broadcast(g, shape, bshape):
    rng = np.random.default_rng(shape[0])
    a, b = activations(rng, shape), activations(rng, bshape)
    assert bits_equal(g.add(a, b), orc_glue.add(a, b))
    assert bits_equal(g.mul(a, b), orc_glue.mul(a, b))


def test_silu_reference_dump(g, nodes):
    for k in range(int(nodes["n_silu"])):
        assert bits_equal(g.silu(nodes[f"silu_{k}_x"], wide=True), nodes[f"silu_{k}_y"]), k


def test_swiglu_reference_dump(g, nodes):
    for k in range(int(nodes["n_swiglu"])):
        _, y = g.silu(nodes[f"swiglu_{k}_x"], wide=True, gate=nodes[f"swiglu_{k}_g"])
        assert bits_equal(y, nodes[f"swiglu_{k}_y"]), k


@pytest.mark.parametrize("wide", [True, False])
@pytest.mark.parametrize("ne0,rows", [(14336, 1), (14336, 16), (11008, 5), (100, 9), (24, 3), (8, 2)])
def test_silu_and_gate(g, ne0, rows, wide):
    rng = np.random.default_rng(ne0 * 3 + rows)
    x = activations(rng, (rows, ne0), scale=2.0)
    x[0, :8] = [0.0, -0.0, 88.0, -88.0, 104.0, -104.0, 1e-30, -1e-30]
    gate = activations(rng, (rows, ne0))
    y, yg = g.silu(x, wide=wide, gate=gate)
    want = orc_glue.silu(x, wide=wide)
    assert bits_equal(y, want)
    assert bits_equal(yg, orc_glue.mul(want, gate))
    assert bits_equal(g.silu(x, wide=wide), want)


def test_rope_reference_dump(g, nodes):
    for k in range(int(nodes["n_rope"])):
        y = g.rope(nodes[f"rope_{k}_x"], nodes[f"rope_{k}_pos"], 16, 2, freq_base=10000.0, n_ctx_orig=512)
        assert bits_equal(y, nodes[f"rope_{k}_y"]), k


@pytest.mark.parametrize("mode", [0, 2])
@pytest.mark.parametrize("ne0,n_dims,heads,toks,base", [(128, 128, 32, 1, 500000.0), (128, 128, 8, 512, 500000.0),
                                                        (128, 64, 4, 7, 10000.0), (64, 64, 6, 33, 1000000.0)])
def test_rope_decoder_sizes(g, mode, ne0, n_dims, heads, toks, base):
    rng = np.random.default_rng(ne0 + toks)
    x = activations(rng, (toks, heads, ne0))
    pos = rng.integers(0, 131072, toks) if toks > 1 else np.array([4095])
    kw = dict(freq_base=base, n_ctx_orig=8192)
    assert bits_equal(g.rope(x, pos, n_dims, mode, **kw), orc_glue.rope(x, pos, n_dims, mode, **kw))


def test_rope_table_indexed_by_device_positions(g):
    m = b200.load()
    rng = np.random.default_rng(21)
    x = activations(rng, (9, 4, 128))
    pos = [0, 1, 2, 511, 3, 100, 4095, 7, 7]
    kw = dict(freq_base=500000.0, n_ctx_orig=8192)
    got = g.rope(x, pos, 128, 0, by_position_rows=4096, **kw)
    assert bits_equal(got, orc_glue.rope(x, pos, 128, 0, **kw))
    assert m.kernel_error() == 0
    g.rope(x, [0, 1, 2, 4096, 3, 100, 4095, 7, 7], 128, 0, by_position_rows=4096, **kw)
    assert m.kernel_error() == 3   # position 4096 is outside a 4096-row table: skipped and reported


def test_rope_table_matches_oracle_with_yarn_and_factors(g):
    kw = dict(freq_base=500000.0, freq_scale=0.25, n_ctx_orig=8192, ext_factor=1.0, attn_factor=1.2, beta_fast=32.0, beta_slow=1.0)
    t = g.rope_table([0, 1, 77, 100000], 128, 128, **kw)
    for i, p in enumerate([0, 1, 77, 100000]):
        assert bits_equal(t[i], orc_glue.rope_cache(p, 128, 128, **kw)), p
    rng = np.random.default_rng(1)
    ff = (1.0 + rng.random(64) * 7).astype(np.float32)
    x = activations(rng, (3, 2, 128))
    got = g.rope(x, [5, 6, 9000], 128, 0, freq_base=500000.0, n_ctx_orig=8192, freq_factors=ff)
    assert bits_equal(got, orc_glue.rope(x, [5, 6, 9000], 128, 0, freq_base=500000.0, n_ctx_orig=8192, freq_factors=ff))


def test_set_rows_reference_dump(g, nodes):
    for k in range(int(nodes["n_set_rows"])):
        x, idx, want = nodes[f"set_rows_{k}_x"], nodes[f"set_rows_{k}_idx"], nodes[f"set_rows_{k}_y"]
        dst = g.set_rows_f16(x, idx, np.zeros((512, x.shape[1]), dtype=np.uint16))
        assert np.array_equal(dst[idx], want.view(np.uint16)), k
        assert not dst[np.setdiff1d(np.arange(512), idx)].any()


def test_set_rows_kv_sizes_and_bad_index(g):
    rng = np.random.default_rng(11)
    x = activations(rng, (16, 1024))
    x[0, :6] = [65504.0, 65520.0, 1e-8, -1e-8, 6.1e-5, np.inf]   # f16 max, overflow to inf, underflow, subnormal edge
    idx = rng.permutation(4096)[:16]
    got = g.set_rows_f16(x, idx, np.full((4096, 1024), 0x1234, dtype=np.uint16))
    want = orc_glue.set_rows_f16(x, idx, np.full((4096, 1024), 0x1234, dtype=np.uint16))
    assert np.array_equal(got, want)
    m = b200.load()
    assert m.kernel_error() == 0
    bad = idx.copy()
    bad[3] = 4096
    got = g.set_rows_f16(x, bad, np.zeros((4096, 1024), dtype=np.uint16))
    assert m.kernel_error() == 2 and m.kernel_error() == 0
    keep = np.delete(np.arange(16), 3)
    assert np.array_equal(got[idx[keep]], want[idx[keep]]) and not got[idx[3]].any()


@pytest.mark.parametrize("ty", [orc.Q4_K, orc.Q6_K, orc.Q8_0, orc.Q4_0, orc.MXFP4])
def test_get_rows_quantized_table(g, ty):
    m = b200.load()
    rng = np.random.default_rng(ty)
    w = rng.standard_normal((200, 512)).astype(np.float32)
    q = orc.quantize_rows(ty, w)
    dev = m.Weight(ty, q, 512)
    ids = [0, 199, 31, 32, 33, 64, 7]
    assert bits_equal(g.get_rows(ty, dev.ptr, 512, 200, ids), orc_glue.get_rows(ty, q, 512, 200, ids))
    assert m.kernel_error() == 0
    g.get_rows(ty, dev.ptr, 512, 200, [0, 200])
    assert m.kernel_error() == 1


def test_get_rows_dense_tables(g):
    m = b200.load()
    rng = np.random.default_rng(2)
    t32 = rng.standard_normal((50, 96)).astype(np.float32)
    d = m.device_array(t32)
    assert bits_equal(g.get_rows(orc.F32, d.ptr, 96, 50, [3, 49, 0]), t32[[3, 49, 0]])
    t16 = t32.astype(np.float16)
    d16 = m.device_array(t16)
    assert bits_equal(g.get_rows(orc.F16, d16.ptr, 96, 50, [3, 49, 0]), t16[[3, 49, 0]].astype(np.float32))


def test_argmax_last_of_equals(g):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((5, 128256)).astype(np.float32)
    x[1, [17, 90000]] = 9.0
    x[2, :] = -np.inf
    x[3, 5] = np.nan
    x[4, :] = np.nan
    got = g.argmax(x)
    want = [orc_glue.argmax(r) for r in x]
    assert list(got) == want and got[1] == 90000 and got[2] == 128255 and got[4] == 0


def q8_K_parts(x, m4):
    """the oracle's Q8_K blocks of each row as (qs, d, bsums): rows below m4 by the 4x8 rule, the rest plain"""
    m, k = x.shape
    qs, d, bs = np.empty((m, k), np.int8), np.empty((m, k // 256), np.float32), np.empty((m, k // 16), np.int16)
    if m4:
        blocks = orc.quantize_q8_K_4x8(x[:m4])        # [m4/4 groups] of block_q8_Kx4: d[4] f32, qs[1024] (8-byte interleave), bsums[64]
        g = blocks.reshape(m4 // 4, k // 256, 4 * 292)
        for r in range(m4):
            grp, lane = r // 4, r % 4
            for b in range(k // 256):
                raw = g[grp, b]
                d[r, b] = raw[:16].view(np.float32)[lane]
                q = raw[16:16 + 1024].view(np.int8).reshape(32, 4, 8)[:, lane, :].reshape(256)
                qs[r, b * 256:(b + 1) * 256] = q
                bs[r, b * 16:(b + 1) * 16] = q.reshape(16, 16).sum(axis=1)
    for r in range(m4, m):
        blk = orc.quantize_q8_K(x[r]).reshape(k // 256, 292)
        d[r] = blk[:, :4].copy().view(np.float32).ravel()
        qs[r] = blk[:, 4:260].copy().view(np.int8).ravel()
        bs[r] = blk[:, 260:292].copy().view(np.int16).ravel()
    return qs, d, bs


@pytest.mark.parametrize("rows,kind", [(1, 2), (3, 2), (8, 3), (7, 4), (16, 4), (37, 2), (64, 3), (45, 4)])
def test_rms_norm_and_silu_leave_q8_K_activations(g, rows, kind):
    """up to 32 rows: one CTA per 256-element block; above: one CTA per row (norm), one warp per block (silu)"""
    m = b200.load()
    rng = np.random.default_rng(rows * 10 + kind)
    m4 = 0 if kind == 2 else rows if kind == 3 else rows - rows % 4
    x = activations(rng, (rows, 1024))
    w = (1.0 + 0.1 * rng.standard_normal(1024)).astype(np.float32)
    y, yw, (qs, d, bs) = g.rms_norm_q8(x, 1e-5, w, kind)
    want = orc_glue.mul(orc_glue.rms_norm(x, 1e-5), w[None, :])
    assert bits_equal(y, orc_glue.rms_norm(x, 1e-5)) and bits_equal(yw, want)
    wq, wd, wb = q8_K_parts(want, m4)
    assert np.array_equal(qs, wq) and bits_equal(d, wd) and np.array_equal(bs, wb)
    gate = activations(rng, (rows, 1024))
    wide = bool(m.lib.b200_host_silu_is_wide())
    s, sg, (qs, d, bs) = g.silu_q8(x, gate, wide, kind)
    want = orc_glue.mul(orc_glue.silu(x, wide=wide), gate)
    assert bits_equal(sg, want)
    wq, wd, wb = q8_K_parts(want, m4)
    assert np.array_equal(qs, wq) and bits_equal(d, wd) and np.array_equal(bs, wb)
