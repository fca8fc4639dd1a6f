"""CUDA path vs the CPU oracle, through the C ABI (-m gpu).

Bars: dequantized weights and Q8 activation blocks bit-exact; mat-mul outputs of
the decode-shaped kernels bit-exact with the CPU route they mirror (which is well
inside the 1e-5 per-element tolerance asked of MUL_MAT).
"""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu

ALL_TYPES = [orc.Q4_K, orc.Q6_K, orc.Q8_0, orc.Q4_0, orc.MXFP4]


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0, "no CUDA device"
    mod.set_device(0)
    return mod


@pytest.mark.parametrize("ty", ALL_TYPES, ids=lambda t: orc.TYPE_NAMES[t])
@pytest.mark.parametrize("shape", [(64, 512), (40, 256), (8, 1024), (1, 256)], ids=str)
def test_tile_layout_round_trip_and_dequantize(dev, ty, shape):
    """upload -> download gives the ggml bytes back; dequantizing from the tile layout equals
    dequantize_row of the original bytes (ragged last tile included)."""
    n, k = shape
    W = synth.weights(ty, n, k, seed=3)
    w = dev.Weight(ty, W, k)
    assert np.array_equal(w.download(), W)
    assert bits_equal(w.dequantize(), orc.dequantize(ty, W, k))


def test_dequantize_golden_blocks(dev, golden):
    """The reference's own block bytes (quantizer output and the hand-built MXFP4 blocks that sweep
    every exponent and code) dequantize on the device to the reference's floats."""
    g = golden("quants")
    names = {"Q4_0": orc.Q4_0, "Q8_0": orc.Q8_0, "Q4_K": orc.Q4_K, "Q6_K": orc.Q6_K, "MXFP4": orc.MXFP4}
    seen = 0
    for key in sorted({k.rsplit("/", 1)[0] for k in g.files}):
        name, kind, n, _ = key.split("/")
        n = int(n)
        if name not in names or n % 256:
            continue
        q, deq = g[key + "/q"], g[key + "/deq"]
        w = dev.Weight(names[name], q.reshape(1, -1), n)
        got = w.dequantize().ravel()
        same = (got.view(np.uint32) == deq.view(np.uint32)) | (np.isnan(got) & np.isnan(deq))
        assert same.all(), key
        seen += 1
    assert seen >= 6


@pytest.mark.parametrize("kind", ["q8_0", "q8_K", "q8_K_4x8"])
@pytest.mark.parametrize("shape", [(1, 4096), (4, 256), (8, 1024), (12, 14336), (40, 1024), (68, 512)], ids=str)  # above 32 rows: the warp-per-block kernels
def test_activation_blocks_bit_exact(dev, kind, shape):
    m, k = shape
    x = synth.activations(m, k, seed=11)
    # rows that exercise the rules' corners: all zero, a negative maximum, a tie for the maximum
    x[0, :256] = 0.0
    if m > 1:
        x[1, 5] = -9.5
        x[1, 77] = 9.5
    if m > 2:
        x[2, 300 % k] = 7.25
        x[2, 10] = -7.25
    if kind == "q8_0":
        assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_0, x), orc.quantize_q8_0(x).ravel())
    elif kind == "q8_K":
        assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_K, x), orc.quantize_q8_K(x).ravel())
    else:
        if m % 4:
            pytest.skip("the 4x8 form takes groups of 4 rows")
        assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_K_4X8, x), orc.quantize_q8_K_4x8(x))


def test_activation_blocks_golden(dev, golden):
    g = golden("repack")
    assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_K, g["Q4_K/gemv_act"]), g["Q4_K/act_plain_q"])
    assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_K_4X8, g["Q4_K/gemm_act"]), g["Q4_K/act_x4_q"])
    rt = golden("real_tensors")
    assert np.array_equal(dev.quantize_activations(dev.ACT_Q8_K, rt["q4k_goss/act"]), rt["q4k_goss/q8k"])


GEMV_SHAPES = [(32, 256), (64, 512), (4096, 4096), (1024, 14336), (96, 2048), (40, 1024), (8, 256)]


@pytest.mark.parametrize("shape", GEMV_SHAPES, ids=str)
@pytest.mark.parametrize("m", [1, 2, 3])
def test_q4_K_decode_mat_mul_bit_exact(dev, shape, m):
    """Q4_K with n % 8 == 0 and fewer than 4 activation rows: the CPU runs its 8x8 gemv on
    plain Q8_K rows (crates/ggml/src/compute.rs:5322, repack.rs:1638)."""
    n, k = shape
    W = synth.weights(orc.Q4_K, n, k, seed=5)
    x = synth.activations(m, k, seed=6)
    want, route = orc.mul_mat(orc.Q4_K, W, x)
    assert route == orc.ROUTE_REPACK
    got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x)
    assert bits_equal(got, want)


def test_q4_K_golden_real_tensor(dev, golden):
    """gpt-oss attn_output Q4_K [4096 x 8] x 3 columns, the reference's production output."""
    rt = golden("real_tensors")
    for key in ("q4k_goss", "q4k_granite"):
        ty, n, rows, cols, flags = (int(v) for v in rt[key + "/hdr"])
        got = dev.mul_mat(dev.Weight(ty, rt[key + "/W"], n), rt[key + "/act"])
        assert bits_equal(got.ravel(), rt[key + "/repack_out"]), key


def test_q4_K_golden_8x8_gemv(dev, golden):
    g = golden("repack")
    n, nrows, nr_gemv, nr_gemm, nc = (int(v) for v in g["Q4_K/dims"])
    got = dev.mul_mat(dev.Weight(orc.Q4_K, g["Q4_K/src"].reshape(nrows, -1), n), g["Q4_K/gemv_act"])
    assert bits_equal(got.ravel(), g["Q4_K/gemv_out"])


def test_q4_K_full_size_periodic_rows(dev):
    """128256 x 4096 (the lm_head shape): rows repeat with period 4096, so must the outputs, and
    the first period equals the oracle."""
    n, k, period = 128256, 4096, 4096
    W = synth.weights(orc.Q4_K, n, k, seed=9, period=period)
    x = synth.activations(1, k, seed=10)
    got = dev.mul_mat(dev.Weight(orc.Q4_K, W, k), x).ravel()
    want, _ = orc.mul_mat(orc.Q4_K, W[:period], x)
    assert bits_equal(got[:period], want.ravel())
    reps = n // period
    assert np.array_equal(got[:reps * period].reshape(reps, period).view(np.uint32),
                          np.tile(want.ravel().view(np.uint32), (reps, 1)))
    assert bits_equal(got[reps * period:], want.ravel()[:n - reps * period])


def test_streaming_kernel_many_launches_no_wait_expired(dev):
    """Back-to-back launches of the bulk-copy streaming kernel (the second launch starts its weight
    prefetch while the first still runs); all bit-exact, and no bounded wait ran out."""
    n, k = 4096, 4096
    W = synth.weights(orc.Q4_K, n, k, seed=33, period=1024)
    w = dev.Weight(orc.Q4_K, W, k)
    xs = [synth.activations(1, k, seed=100 + i) for i in range(3)]
    dxs = [dev.device_array(x) for x in xs]
    outs = [dev.DeviceBuffer(4 * n) for _ in xs]
    dev.lib.b200_debug_stream_wait(1 << 20, -1)   # select the streaming kernel (the normal poll limit, nothing skipped)
    try:
        for _ in range(5):
            for dx, do in zip(dxs, outs):
                dev.mul_mat_device(w, dx, 1, do)
        dev.synchronize()
    finally:
        dev.lib.b200_debug_stream_wait(0, -1)
    assert dev.kernel_error() == 0
    for x, do in zip(xs, outs):
        want, _ = orc.mul_mat(orc.Q4_K, W, x)
        assert bits_equal(do.download(np.float32, n), want.ravel())


def test_empty_and_refused_shapes(dev):
    W = synth.weights(orc.Q4_K, 32, 256)
    w = dev.Weight(orc.Q4_K, W, 256)
    out = dev.mul_mat(w, np.zeros((0, 256), dtype=np.float32))
    assert out.shape == (0, 32)
    # all-zero activations give exact zeros
    z = dev.mul_mat(w, np.zeros((1, 256), dtype=np.float32))
    assert not z.any()


# (type, route the reference takes, allowed m) for the other decode-shaped kernels
OTHER_DECODE = [
    (orc.Q6_K, orc.ROUTE_ROWDOT, [1, 2, 7]),     # row dot below 8 activation rows (compute.rs:1596)
    (orc.Q8_0, orc.ROUTE_ROWDOT, [1, 3]),        # row dot; tinyBLAS gives the same values
    (orc.Q4_0, orc.ROUTE_REPACK, [1, 2, 3]),     # 8x8 gemv == gemm per element
    (orc.MXFP4, orc.ROUTE_REPACK, [1, 2, 5]),    # 8x8 gemv per activation row
]


@pytest.mark.parametrize("case", OTHER_DECODE, ids=lambda c: orc.TYPE_NAMES[c[0]])
@pytest.mark.parametrize("shape", [(32, 256), (64, 512), (4096, 4096), (512, 14336), (40, 1024)], ids=str)
def test_other_types_decode_mat_mul_bit_exact(dev, case, shape):
    ty, route, ms = case
    n, k = shape
    W = synth.weights(ty, n, k, seed=15)
    w = dev.Weight(ty, W, k)
    for m in ms:
        x = synth.activations(m, k, seed=16 + m)
        want, r = orc.mul_mat(ty, W, x)
        assert r == route
        assert bits_equal(dev.mul_mat(w, x), want), f"m={m}"


def test_golden_real_tensors_q6_K_and_mxfp4_blocks(dev, golden):
    rt = golden("real_tensors")
    ty, n, rows, cols, flags = (int(v) for v in rt["q6k_granite/hdr"])
    got = dev.mul_mat(dev.Weight(ty, rt["q6k_granite/W"], n), rt["q6k_granite/act"])
    assert bits_equal(got, rt["q6k_granite/plain_out"])
    # the reference's hand-built MXFP4 blocks (every exponent, every code), tiled to 8 rows of 1024
    q = golden("quants")
    key = [k for k in q.files if k.startswith("MXFP4/raw/1024") and k.endswith("/q")][0]
    W = np.tile(q[key].reshape(1, -1), (8, 1))
    x = (synth.activations(1, 1024, seed=40) * 1e-3).astype(np.float32)
    want, route = orc.mul_mat(orc.MXFP4, W, x)
    assert route == orc.ROUTE_REPACK
    got = dev.mul_mat(dev.Weight(orc.MXFP4, W, 1024), x)
    same = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert same.all()


# ---- batched mat-mul: every route the reference takes for m >= 4 --------------------------------
BATCHED = [
    # (type, n, k, m, route)
    (orc.Q4_K, 64, 512, 4, orc.ROUTE_REPACK),     # one 4-row group: 8x8 gemm numerics
    (orc.Q4_K, 96, 1024, 9, orc.ROUTE_REPACK),    # two groups + a gemv tail row
    (orc.Q4_K, 4096, 4096, 32, orc.ROUTE_REPACK),
    (orc.Q4_K, 36, 512, 8, orc.ROUTE_TILED),      # rows not a multiple of 8: tiled from 8 columns on
    (orc.Q4_K, 36, 512, 3, orc.ROUTE_ROWDOT),     # ... and the row dot below
    (orc.Q6_K, 64, 512, 8, orc.ROUTE_TILED),
    (orc.Q6_K, 1024, 4096, 33, orc.ROUTE_TILED),
    (orc.Q8_0, 64, 512, 8, orc.ROUTE_ROWDOT),
    (orc.Q4_0, 64, 512, 12, orc.ROUTE_REPACK),
    (orc.MXFP4, 768, 2048, 8, orc.ROUTE_REPACK),
]


@pytest.mark.parametrize("case", BATCHED, ids=lambda c: f"{orc.TYPE_NAMES[c[0]]}-{c[1]}x{c[2]}-m{c[3]}")
def test_batched_mat_mul_bit_exact(dev, case):
    ty, n, k, m, route = case
    W = synth.weights(ty, n, k, seed=51)
    x = synth.activations(m, k, seed=52)
    want, r = orc.mul_mat(ty, W, x)
    assert r == route
    assert bits_equal(dev.mul_mat(dev.Weight(ty, W, k), x), want)


def test_golden_8x8_gemm_and_tiled_outputs(dev, golden):
    g = golden("repack")
    n, nrows, nr_gemv, nr_gemm, nc = (int(v) for v in g["Q4_K/dims"])
    got = dev.mul_mat(dev.Weight(orc.Q4_K, g["Q4_K/src"].reshape(nrows, -1), n), g["Q4_K/gemm_act"])
    assert bits_equal(got, g["Q4_K/gemm_out"])
    t = golden("tiled")
    names = {"Q4_K": orc.Q4_K, "Q6_K": orc.Q6_K}
    for name, ty in names.items():
        for shape in ("300x40", "300x12", "12x8", "188x300"):
            key = f"mm/{name}/{shape}"
            X = t[key + "/X"]
            got = dev.mul_mat(dev.Weight(ty, t[key + "/W"], X.shape[1]), X)
            assert bits_equal(got, t[key + "/dst"]), key


def test_k_split_kernel_passes_the_same_cases():
    """B200_GEMV_KSPLIT=1 (read once per process) splits K of the few-tile decode mat-muls over several CTAs, the
    last arriver running the chain: run the Q4_K decode tests of this file in a child with it set"""
    import os
    import subprocess
    import sys
    if os.environ.get("B200_GEMV_KSPLIT") == "1":
        pytest.skip("already the child")
    env = dict(os.environ, B200_GEMV_KSPLIT="1")
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider", "-k", "q4_K or streaming"],
                       env=env, capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
