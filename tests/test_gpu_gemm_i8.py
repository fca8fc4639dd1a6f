"""Prompt-shaped mat-muls of Q6_K, Q4_0, MXFP4 and Q8_0 weights on the tcgen05 int8 kernels (-m gpu).

Q6_K (tiled route), Q4_0 and MXFP4 (8x8 gemm route) must give the CPU oracle's bits: the kernels compute the same
exact integer block dots and run the same f32 chain.  Q8_0's tensor-core form belongs to the library's fast
numerics mode: it adds whole 32-element block dots where the CPU route adds eight lanes of four, so it is held to
the mat-mul tolerance instead, defined as the reference defines it (crates/ggml/src/compute.rs:7467-7577):
|got - ref| <= 1e-5 * sum_k |w_k x_k| per output element."""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu

SHAPES = [(256, 1024, 40), (128, 256, 32), (300, 2048, 33), (1024, 4096, 100), (4096, 4096, 512), (96, 512, 8)]


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("ty", [orc.Q6_K, orc.Q4_0, orc.MXFP4], ids=lambda t: orc.TYPE_NAMES[t])
def test_bit_exact_types(dev, ty, shape, monkeypatch):
    n, k, m = shape
    if ty != orc.Q6_K and n % 8:
        pytest.skip("the 8x8 route needs rows % 8 == 0")
    W = synth.weights(ty, n, k, seed=400 + ty, period=512)
    x = synth.activations(m, k, seed=401 + m)
    want, _ = orc.mul_mat(ty, W, x)
    # Q6_K takes its tcgen05 kernel only on request (the mma.sync kernel is the quicker one): ask for it here
    monkeypatch.setenv("B200_Q6K_TCGEN05", "1")
    got = dev.mul_mat(dev.Weight(ty, W, k), x)
    assert dev.kernel_error() == 0
    assert bits_equal(got, want), f"max |d| = {np.abs(got - want).max()}"


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_q8_0_fast_mode_within_the_mat_mul_tolerance(dev, shape):
    n, k, m = shape
    W = synth.weights(orc.Q8_0, n, k, seed=410, period=512)
    x = synth.activations(m, k, seed=411 + m)
    want, _ = orc.mul_mat(orc.Q8_0, W, x)
    dev.set_numerics(dev.FAST)
    try:
        got = dev.mul_mat(dev.Weight(orc.Q8_0, W, k), x)
    finally:
        dev.set_numerics(dev.EXACT)
    assert dev.kernel_error() == 0
    bound = 1e-5 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q8_0, W, k)).astype(np.float64).T)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert (err <= bound).all(), f"worst ratio to the bound: {(err / bound).max():.3g}"
    print(f"Q8_0 {shape}: max |got - ref| / sum|w x| = {(err / (bound * 1e5)).max():.2e}")
    # and in exact mode the same call reproduces the CPU's lanes
    assert bits_equal(dev.mul_mat(dev.Weight(orc.Q8_0, W, k), x), want)
