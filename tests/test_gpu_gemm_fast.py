"""Q4_K prompt mat-muls in the library's fast numerics mode (csrc/gemm_tcgen05_fast.cu) against the CPU oracle (-m gpu).

The kernel accumulates a whole super-block on the tensor cores and applies the block scales once per super-block, where
the CPU routes (8x8 gemm chain: crates/ggml/src/repack.rs:1692-1768; tiled chain: tiled.rs) run fused multiply-adds
per sub-block pair.  It is held to the mat-mul tolerance, defined as the reference defines it
(crates/ggml/src/compute.rs:7467-7577): |got - ref| <= 1e-5 * sum_k |w_k x_k| per output element; in exact mode
the same call gives the CPU's bits."""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu

# (weight rows, row length, activation rows): ragged row blocks and column blocks, one and many super-blocks,
# row counts that take the tiled route (n % 8 != 0) and the 8x8 route, the benchmark's square shape
SHAPES = [(128, 256, 64), (256, 1024, 67), (296, 2048, 100), (300, 512, 129), (1024, 4096, 200), (4096, 4096, 512), (520, 14336, 256)]


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


def pick_kernel(monkeypatch, form):
    """128 or 256 activation rows per CTA; "/n": n CTAs instead of one per SM, so that the runs of (tile, super-block) units
    cut the tiles in other places (partial tiles through the workspace, several CTAs per tile, several tiles per CTA)"""
    cols, _, ctas = form.partition("/")
    monkeypatch.setenv("B200_GEMM_FAST_COLS", cols)
    if ctas:
        monkeypatch.setenv("B200_GEMM_FAST_CTAS", ctas)


FORMS = ["128", "256", "256/7", "128/37", "256/3"]


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_q4_K_fast_mode_within_the_mat_mul_tolerance(dev, shape, form, monkeypatch):
    n, k, m = shape
    pick_kernel(monkeypatch, form)
    monkeypatch.setenv("B200_GEMM_FAST", "2")   # the fast kernel whatever the row count
    W = synth.weights(orc.Q4_K, n, k, seed=420, period=512)
    x = synth.activations(m, k, seed=421 + m)
    want, _ = orc.mul_mat(orc.Q4_K, W, x)
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    assert dev.kernel_error() == 0
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q4_K, W, k)).astype(np.float64).T)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    print(f"Q4_K {shape}: max |got - ref| / sum|w x| = {(err / (bound * 1e5)).max():.2e}")
    assert (err <= bound).all(), f"worst ratio to the bound: {(err / bound).max():.3g}"
    assert n * m < 1 << 14 or not bits_equal(got, want), "the fast kernel was not taken"
    # and in exact mode the same call reproduces the CPU's chain
    assert bits_equal(dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x), want)


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_q6_K_fast_mode_within_the_mat_mul_tolerance(dev, shape, form, monkeypatch):
    """Q6_K on the same kernel: a weight s (q - 32) goes in as two exact f16 operands, s (8 (q >> 3) - 32) and s (q & 7)
    (tiled chain on the CPU: crates/ggml/src/tiled.rs:723-839)"""
    n, k, m = shape
    pick_kernel(monkeypatch, form)
    monkeypatch.setenv("B200_GEMM_FAST", "2")   # the fast kernel whatever the row count
    W = synth.weights(orc.Q6_K, n, k, seed=450, period=512)
    x = synth.activations(m, k, seed=451 + m)
    want, _ = orc.mul_mat(orc.Q6_K, W, x)
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q6_K, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    assert dev.kernel_error() == 0
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q6_K, W, k)).astype(np.float64).T)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    print(f"Q6_K {shape}: max |got - ref| / sum|w x| = {(err / (bound * 1e5)).max():.2e}")
    assert (err <= bound).all(), f"worst ratio to the bound: {(err / bound).max():.3g}"
    assert bits_equal(dev.mul_mat(dev.Weight(orc.Q6_K, W, k), x), want)


def test_q6_K_fast_mode_extreme_scales(dev, monkeypatch):
    """scales of -128 and 127 against quants of 0 and 63: the largest products the two operand parts have to carry"""
    monkeypatch.setenv("B200_GEMM_FAST", "2")
    n, k, m = 128, 512, 64
    W = synth.weights(orc.Q6_K, n, k, seed=460).copy()
    blocks = W.reshape(n, k // 256, 210)      # ql[128] qh[64] scales[16] d
    blocks[0, 0, 192:208] = np.array([-128, 127] * 8, dtype=np.int8).view(np.uint8)
    blocks[0, 0, 0:128] = 0xFF                # low nibbles 15 ...
    blocks[0, 0, 128:192] = 0xFF              # ... high bits 3: q = 63
    blocks[1, 1, 192:208] = np.array([127, -128] * 8, dtype=np.int8).view(np.uint8)
    blocks[1, 1, 0:192] = 0                   # q = 0
    x = synth.activations(m, k, seed=461)
    want, _ = orc.mul_mat(orc.Q6_K, W, x)
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q6_K, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q6_K, W, k)).astype(np.float64).T)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= bound).all(), f"worst ratio to the bound: {(err / bound).max():.3g}"


@pytest.mark.parametrize("form", FORMS)
def test_q4_K_fast_mode_blocks_with_odd_scales(dev, form, monkeypatch):
    """super-blocks whose d is zero, tiny against dmin (the ratio would leave the f16 range), or negative: the kernel takes
    their mins on the CUDA cores; both column widths of the kernel"""
    n, k, m = 264, 1536, 200
    W = synth.weights(orc.Q4_K, n, k, seed=440, period=512).copy()
    blocks = W.reshape(n, k // 256, 144)
    d = blocks[:, :, 0:2].view(np.float16)
    dmin = blocks[:, :, 2:4].view(np.float16)
    d[3, 1] = 0.0
    d[3, 4] = 0.0
    dmin[3, 4] = 0.0
    d[40, 0] = np.float16(6e-8)         # the smallest subnormal against an ordinary dmin
    d[129, 5] = -d[129, 5]
    dmin[200, 2] = -dmin[200, 2]
    d[263, :] = 0.0
    x = synth.activations(m, k, seed=441)
    want, _ = orc.mul_mat(orc.Q4_K, W, x)
    pick_kernel(monkeypatch, form)
    monkeypatch.setenv("B200_GEMM_FAST", "2")
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    assert dev.kernel_error() == 0
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q4_K, W, k)).astype(np.float64).T)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= bound + 1e-30).all(), f"worst ratio to the bound: {(err / np.maximum(bound, 1e-30)).max():.3g}"


def test_q4_K_fast_mode_switch(dev, monkeypatch):
    """B200_GEMM_FAST=0 keeps the exact kernels under the fast policy too"""
    n, k, m = 256, 1024, 64
    W = synth.weights(orc.Q4_K, n, k, seed=430, period=512)
    x = synth.activations(m, k, seed=431)
    want, _ = orc.mul_mat(orc.Q4_K, W, x)
    monkeypatch.setenv("B200_GEMM_FAST", "0")
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    assert bits_equal(got, want)
