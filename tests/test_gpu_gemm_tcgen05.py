"""The tcgen05 prompt mat-mul (Q4_K, 32 activation rows and up) against the CPU oracle and against the
decode-shaped kernels: same chains, so every output has to agree bit for bit.  The whole file runs with the
library choosing between the integer and the two-pass kernel by size (the default) and, in child processes with
B200_GEMM_TCGEN05_F16=0 .. 4, on each kernel alone: the integer one, the f16-operand ones with 32 and 64 activation
rows per CTA that convert their own operands, and the two-pass ones (64 and 128 activation rows per CTA)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0, "no CUDA device"
    mod.set_device(0)
    return mod


CASES = [
    # (n, k, m, route)
    (128, 256, 32, orc.ROUTE_REPACK),    # one CTA, one super-block: a single pipeline step
    (128, 1024, 32, orc.ROUTE_REPACK),   # four steps: stage and accumulator rings wrap
    (160, 2048, 45, orc.ROUTE_REPACK),   # rows: a partly filled 128-row block; columns: 44 by the gemm chain + 1 tail row
    (256, 512, 96, orc.ROUTE_REPACK),
    (36, 512, 40, orc.ROUTE_TILED),      # rows not a multiple of 8: tiled chain; 36 rows of a 128-row block
    (300, 768, 64, orc.ROUTE_TILED),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c[0]}x{c[1]}-m{c[2]}")
def test_against_the_oracle(dev, case):
    n, k, m, route = case
    W = synth.weights(orc.Q4_K, n, k, seed=61)
    x = synth.activations(m, k, seed=62)
    want, r = orc.mul_mat(orc.Q4_K, W, x)
    assert r == route
    got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    assert dev.kernel_error() == 0
    assert bits_equal(got, want), f"max |d| = {np.abs(got - want).max()}"


@pytest.mark.parametrize("shape", [(4096, 4096, 512), (1024, 14336, 200)], ids=str)
def test_full_size_columns_agree_with_four_column_calls(dev, shape):
    """512 activation rows in one call (tcgen05) = the same rows four at a time (the decode-shaped gemm kernel)"""
    n, k, m = shape
    W = synth.weights(orc.Q4_K, n, k, seed=63)
    x = synth.activations(m, k, seed=64)
    w = dev.Weight(orc.Q4_K, W, k)
    whole = dev.mul_mat(w, x)
    assert dev.kernel_error() == 0
    for c0 in list(range(0, m, 52))[:6] + [m - 4]:
        part = dev.mul_mat(w, x[c0:c0 + 4])
        assert bits_equal(whole[c0:c0 + 4], part), f"columns {c0}..{c0 + 3}"


@pytest.mark.parametrize("signs", ["same", "random"])
def test_largest_integers_stay_exact(dev, signs):
    """every scale and min 63, every nibble 15, every activation byte +-127: the pair sums reach
    2 * 32 * 15 * 127 * 63 = 7.68e6, the largest integers the f16 operands / f32 accumulators have to carry"""
    n, k, m = 128, 1024, 32
    blk = np.zeros(144, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    blk[4:] = 0xFF
    W = np.tile(blk, (n, k // 256))
    rng = np.random.default_rng(71)
    x = np.full((m, k), -3.0, dtype=np.float32)
    if signs == "random":
        x *= rng.choice([-1.0, 1.0], size=x.shape).astype(np.float32)
        W = W.copy().reshape(n, k // 256, 144)
        W[:, :, 16:] = rng.choice([0xFF, 0xF0, 0x0F, 0xFE], size=(n, k // 256, 128)).astype(np.uint8)
        W = W.reshape(n, -1)
    want, r = orc.mul_mat(orc.Q4_K, W, x)
    assert r == orc.ROUTE_REPACK
    got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    assert dev.kernel_error() == 0
    assert bits_equal(got, want), f"max |d| = {np.abs(got - want).max()}"


@pytest.mark.parametrize("choice", ["0", "1", "2", "3", "4"])
def test_f16_operand_kernels_pass_the_same_cases(choice):
    """the library reads B200_GEMM_TCGEN05_F16 once per process: run this file's other tests in a child with it set"""
    if os.environ.get("B200_GEMM_TCGEN05_F16") in ("0", "1", "2", "3", "4"):
        pytest.skip("already the child")
    env = dict(os.environ, B200_GEMM_TCGEN05_F16=choice)
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"], env=env,
                       capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


SMALL_CASES = [
    # (n, k, m): 8 to 31 activation rows take the K-split mma kernel (gemm chain)
    (64, 512, 8), (96, 1024, 9), (4096, 4096, 16), (1024, 14336, 16), (160, 2304, 31), (4096, 4096, 13),
]


@pytest.mark.parametrize("case", SMALL_CASES, ids=lambda c: f"{c[0]}x{c[1]}-m{c[2]}")
def test_small_batches_against_the_oracle_and_four_column_calls(dev, case):
    n, k, m = case
    W = synth.weights(orc.Q4_K, n, k, seed=65, period=256)
    x = synth.activations(m, k, seed=66)
    w = dev.Weight(orc.Q4_K, W, k)
    got = dev.mul_mat(w, x)
    assert dev.kernel_error() == 0
    if n * k <= 1 << 22:
        want, r = orc.mul_mat(orc.Q4_K, W, x)
        assert r == orc.ROUTE_REPACK
        assert bits_equal(got, want), f"max |d| = {np.abs(got - want).max()}"
    m4 = m - m % 4
    for c0 in range(0, m4, 4):
        assert bits_equal(got[c0:c0 + 4], dev.mul_mat(w, x[c0:c0 + 4])), f"columns {c0}..{c0 + 3}"


@pytest.mark.parametrize("case", [(64, 512, 8), (1024, 4096, 16), (300, 1024, 31), (96, 14336, 12)], ids=str)
def test_q6_K_small_batches_against_the_oracle(dev, case):
    n, k, m = case
    W = synth.weights(orc.Q6_K, n, k, seed=67, period=128)
    x = synth.activations(m, k, seed=68)
    want, r = orc.mul_mat(orc.Q6_K, W, x)
    assert r == orc.ROUTE_TILED
    got = dev.mul_mat(dev.Weight(orc.Q6_K, W, k), x)
    assert bits_equal(got, want), f"max |d| = {np.abs(got - want).max()}"
