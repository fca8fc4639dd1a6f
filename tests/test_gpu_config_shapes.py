"""The benchmark configurations' own shapes against the CPU oracle (-m gpu).

Quantized mat-mul sweep: weight types Q4_K, Q6_K, Q8_0 and MXFP4, weight shapes 14336 x 4096, 4096 x 14336 and
128256 x 4096, 512 and 2048 activation rows.  The weight matrices repeat a block of distinct rows (every output
row depends on its own weight row only, and each of these row counts keeps the reference's route: a multiple of
8), so the oracle computes one period and the rest of the GPU result must repeat it bit for bit.  FLASH_ATTN_EXT:
512 query rows over 32768 cached positions, 32 query heads on 8 KV heads of 128.
Everything is compared bit for bit: these are the reference's routes' own f32 chains.
"""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal
from test_gpu_flash_attn import synth_case

pytestmark = pytest.mark.gpu

PERIOD = 256
TYPES = [orc.Q4_K, orc.Q6_K, orc.Q8_0, orc.MXFP4]
SHAPES = [(14336, 4096), (4096, 14336), (128256, 4096)]


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


def mul_mat_device(dev, w, x):
    """device-resident activations and result: the result of the largest case is 1 GB"""
    m, k = x.shape
    dx = dev.device_array(x)
    out = dev.DeviceBuffer(4 * m * w.n_rows)
    dev.mul_mat_device(w, dx, m, out)
    dev.synchronize()
    assert dev.kernel_error() == 0
    return out.download(np.float32, m * w.n_rows).reshape(m, w.n_rows)


@pytest.mark.parametrize("m", [512, 2048])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("ty", TYPES, ids=lambda t: orc.TYPE_NAMES[t])
def test_sweep_shape_matches_the_oracle(dev, ty, shape, m):
    n, k = shape
    W = synth.weights(ty, n, k, seed=300 + ty, period=PERIOD)
    x = synth.activations(m, k, seed=301 + m)
    want, _ = orc.mul_mat(ty, W[:PERIOD], x)              # [m, PERIOD]: 256 rows take the same route as n rows (both % 8 == 0)
    got = mul_mat_device(dev, dev.Weight(ty, W, k), x)    # [m, n]
    assert bits_equal(got[:, :PERIOD], want), f"max |d| = {np.abs(got[:, :PERIOD] - want).max()}"
    reps = n // PERIOD
    tiled = got[:, :reps * PERIOD].reshape(m, reps, PERIOD).view(np.uint32)
    assert (tiled == want.view(np.uint32)[:, None, :]).all(), "a later period of rows differs from the first"
    tail = n - reps * PERIOD
    if tail:
        assert bits_equal(got[:, reps * PERIOD:], want[:, :tail])


def test_prefill_512_rows_over_32768_positions(dev):
    q, k, v, mask = synth_case(32, 8, 128, 512, 32768, seed=3276)
    want, path = orc.flash_attn(q, k, v, mask, 1.0 / np.sqrt(128.0))
    assert path == orc.FA_TILED
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 1.0 / np.sqrt(128.0))
    assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
    assert bits_equal(got, want)
