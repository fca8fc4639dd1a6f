"""The oracle's vector bodies (oracle/oracle_simd.cpp: AVX2 and AVX-512 VNNI) against its scalar loops.

The reference states that its SIMD kernels and their scalar specifications give identical bits
(crates/ggml/src/repack.rs:1777-, crates/ggml/src/simd_x86.rs:799): the integer sub-dots are exact and the f32
chain is the same sequence of fused multiply-adds.  The same must hold here, at every level the host offers, on
ordinary data, on worst-case magnitudes (all nibbles 15 / all six-bit values 63 against quants of -128 and 127,
where a 16-bit intermediate would be closest to overflow) and through the golden vectors (which run at the
default level in test_oracle_golden.py).
"""
import numpy as np
import pytest

import orc
import synth
from conftest import bits_equal


@pytest.fixture
def levels():
    orc.set_simd(2)
    top = orc.simd_level()
    yield list(range(top + 1))
    orc.set_simd(2)


def run_levels(levels, fn):
    outs = []
    for lv in levels:
        orc.set_simd(lv)
        assert orc.simd_level() == lv
        outs.append(fn())
    return outs


@pytest.mark.parametrize("m", [1, 3, 4, 9])
@pytest.mark.parametrize("ty", [orc.Q4_K, orc.Q6_K])
def test_simd_equals_scalar(levels, ty, m):
    n, k = 72, 1024
    W = synth.weights(ty, n, k, seed=11 + m)
    X = synth.activations(m, k, seed=5)
    for route in (orc.ROUTE_AUTO, orc.ROUTE_ROWDOT, orc.ROUTE_REPACK):
        if route == orc.ROUTE_REPACK and ty != orc.Q4_K:
            continue
        outs = run_levels(levels, lambda: orc.mul_mat(ty, W, X, route=route)[0])
        for lv, o in zip(levels[1:], outs[1:]):
            assert bits_equal(o, outs[0]), f"type {ty} m {m} route {route}: level {lv} differs from scalar"
    if len(levels) == 1:
        pytest.skip("host has no AVX2: only the scalar level ran")


@pytest.mark.parametrize("ty", [orc.Q4_K, orc.Q6_K])
def test_simd_extreme_magnitudes(levels, ty):
    """Saturating patterns: the largest weights' codes everywhere, activations that quantize to +-127 / -128."""
    n, k = 16, 512
    rs = orc.row_size(ty, k)
    rng = np.random.default_rng(3)
    W = synth.weights(ty, n, k, seed=2).copy()
    Wb = W.reshape(n, k // 256, rs // (k // 256))
    if ty == orc.Q4_K:
        Wb[:, :, 16:] = 0xFF          # every nibble 15 (block_q4_K: d, dmin, 12 scale bytes, 128 quant bytes)
        Wb[:, :, 4:16] = 0xFF         # the largest six-bit scales and mins
    else:
        Wb[:, :, :192] = 0xFF         # ql and qh: every six-bit value 63 (block_q6_K: ql 128, qh 64, scales 16, d)
        Wb[:, :, 192:208] = rng.choice(np.array([127, 0x80], dtype=np.uint8), size=(n, k // 256, 16))
    for signs in (np.ones(k), -np.ones(k), rng.choice([-1.0, 1.0], size=k)):
        X = np.tile((signs * 1000.0).astype(np.float32), (4, 1))
        outs = run_levels(levels, lambda: orc.mul_mat(ty, W, X)[0])
        for lv, o in zip(levels[1:], outs[1:]):
            assert bits_equal(o, outs[0]), f"type {ty}: level {lv} differs from scalar on saturating input"


def test_simd_level_cap():
    orc.set_simd(0)
    assert orc.simd_level() == 0
    orc.set_simd(7)
    assert orc.simd_level() in (0, 1, 2)
    orc.set_simd(2)
