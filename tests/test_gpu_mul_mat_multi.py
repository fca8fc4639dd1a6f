"""b200_mul_mat_q8_multi: one activation row against several Q4_K matrices in one launch gives, element for
element, what one launch per matrix gives (and so what the CPU route gives)."""
import ctypes as C

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


@pytest.mark.parametrize("rows", [(1024, 1024, 4096), (14336, 14336), (40, 8, 72), (4096,)], ids=str)
def test_multi_equals_single_launches(dev, rows):
    k = 4096 if max(rows) > 100 else 512
    x = synth.activations(1, k, seed=5)
    Ws = [synth.weights(orc.Q4_K, n, k, seed=10 + i, period=64) for i, n in enumerate(rows)]
    ws = [dev.Weight(orc.Q4_K, W, k) for W in Ws]
    dx = dev.device_array(x)
    act = dev.DeviceBuffer(dev.lib.b200_act_scratch_nbytes(1, k))
    dev.check(dev.lib.b200_quantize_activations_device(dev.ACT_Q8_K, 1, k, dx.ptr, k, act.ptr, None), "quantize")
    outs = [dev.DeviceBuffer(4 * n) for n in rows]
    count = len(rows)
    n_arr = (C.c_int64 * count)(*rows)
    w_arr = (C.c_void_p * count)(*[w.ptr for w in ws])
    d_arr = (C.c_void_p * count)(*[o.ptr for o in outs])
    dev.check(dev.lib.b200_mul_mat_q8_multi(orc.Q4_K, C.c_int64(k), count, n_arr, w_arr, C.c_void_p(act.ptr), dev.ACT_Q8_K, d_arr, None), "multi")
    dev.synchronize()
    for W, w, o, n in zip(Ws, ws, outs, rows):
        got = o.download(np.float32, n)
        single = dev.mul_mat(w, x)[0]
        assert bits_equal(got, single)
        if n <= 4096:
            want, _ = orc.mul_mat(orc.Q4_K, W, x)
            assert bits_equal(got, want[0])


def test_refusals(dev):
    n_arr = (C.c_int64 * 1)(36)
    nul = (C.c_void_p * 1)(1)
    rc = dev.lib.b200_mul_mat_q8_multi(orc.Q4_K, C.c_int64(512), 1, n_arr, nul, C.c_void_p(1), dev.ACT_Q8_K, nul, None)
    assert rc != 0 and b"8x8 gemv route" in dev.lib.b200_last_error()
    rc = dev.lib.b200_mul_mat_q8_multi(orc.Q6_K, C.c_int64(512), 1, n_arr, nul, C.c_void_p(1), dev.ACT_Q8_K, nul, None)
    assert rc != 0 and b"Q4_K only" in dev.lib.b200_last_error()


@pytest.mark.parametrize("mode", ["fast", "exact"])
@pytest.mark.parametrize("case", [((1024, 1024, 4096), 4096, 256), ((14336, 14336), 4096, 512), ((4096, 264), 1024, 68), ((520,), 2048, 100),
                                  ((4096, 1024, 1024), 4096, 16), ((14336, 14336), 4096, 12), ((264, 520), 512, 28), ((1024, 1024), 14336, 8)], ids=str)
def test_rows_multi_equals_single_calls(dev, case, mode):
    """b200_mul_mat_q8_rows_multi: several Q4_K matrices against the same prompt batch give what one b200_mul_mat_q8 call
    per matrix gives: bit for bit in the exact numerics mode (the CPU chain's kernels); in the fast mode one launch of the
    tensor-core kernel, whose CTAs cut the tiles' super-block sums in other places than a launch per matrix does, so the
    f32 sums associate differently: held to a tenth of the mode's tolerance of 1e-5 sum |w x|.  A batched decode step's 8 to
    31 rows take the few-rows kernel with the matrices as one grid: the same CTAs and chains, bit-identical in both modes."""
    rows, k, m = case
    x = synth.activations(m, k, seed=6)
    Ws = [synth.weights(orc.Q4_K, n, k, seed=20 + i, period=64) for i, n in enumerate(rows)]
    ws = [dev.Weight(orc.Q4_K, W, k) for W in Ws]
    dx = dev.device_array(x)
    kind = dev.act_kind_for(orc.Q4_K, rows[0], m)
    act = dev.DeviceBuffer(dev.lib.b200_act_scratch_nbytes(m, k))
    dev.check(dev.lib.b200_quantize_activations_device(kind, m, k, dx.ptr, k, act.ptr, None), "quantize")
    outs = [dev.DeviceBuffer(4 * n * m) for n in rows]
    count = len(rows)
    n_arr = (C.c_int64 * count)(*rows)
    ld_arr = (C.c_int64 * count)(*rows)
    w_arr = (C.c_void_p * count)(*[w.ptr for w in ws])
    d_arr = (C.c_void_p * count)(*[o.ptr for o in outs])
    dev.set_numerics(dev.FAST if mode == "fast" else dev.EXACT)
    try:
        dev.check(dev.lib.b200_mul_mat_q8_rows_multi(orc.Q4_K, C.c_int64(k), C.c_int64(m), count, n_arr, w_arr, C.c_void_p(act.ptr), kind, d_arr, ld_arr, None),
                  "rows_multi")
        dev.synchronize()
        assert dev.kernel_error() == 0
        for W, w, o, n in zip(Ws, ws, outs, rows):
            got = o.download(np.float32, n * m).reshape(m, n)
            single = dev.mul_mat(w, x)
            if mode == "exact" or m < 32:
                assert bits_equal(got, single)
            else:
                bound = 1e-6 * (np.abs(x).astype(np.float64) @ np.abs(orc.dequantize(orc.Q4_K, W, k)).astype(np.float64).T)
                assert (np.abs(got.astype(np.float64) - single.astype(np.float64)) <= bound).all()
    finally:
        dev.set_numerics(dev.EXACT)


@pytest.mark.parametrize("case", [(orc.Q4_K, 4096, 4096, 16), (orc.Q4_K, 1032, 512, 28), (orc.Q6_K, 4096, 14336, 16), (orc.Q6_K, 100, 512, 9),
                                  (orc.Q4_K, 4096, 14336, 8)], ids=str)
def test_rows_add_equals_mat_mul_then_add(dev, case):
    """b200_mul_mat_q8_rows_add (the residual ADD of a batched decode step inside the few-rows kernels): dst is what
    b200_mul_mat_q8 gives bit for bit, sum is dst + addend with one rounded f32 add per element, also with the sum written
    over the addend (the residual updated in place) and with row strides larger than the rows."""
    ty, n, k, m = case
    assert dev.lib.b200_mul_mat_q8_rows_add_fusable(ty, C.c_int64(n), C.c_int64(m)) == 1
    x = synth.activations(m, k, seed=11)
    W = synth.weights(ty, n, k, seed=31, period=64)
    w = dev.Weight(ty, W, k)
    kind = dev.act_kind_for(ty, n, m)
    act = dev.DeviceBuffer(dev.lib.b200_act_scratch_nbytes(m, k))
    dx = dev.device_array(x)
    dev.check(dev.lib.b200_quantize_activations_device(kind, m, k, dx.ptr, k, act.ptr, None), "quantize")
    ld = n + 8
    add = np.random.default_rng(5).standard_normal((m, ld)).astype(np.float32)
    dadd = dev.device_array(add)
    dst, dsum = dev.DeviceBuffer(4 * n * m), dev.DeviceBuffer(4 * ld * m)
    dev.check(dev.lib.b200_mul_mat_q8_rows_add(ty, C.c_int64(n), C.c_int64(k), C.c_int64(m), C.c_void_p(w.ptr), C.c_void_p(act.ptr), kind, C.c_void_p(dst.ptr),
                                               C.c_int64(n), C.c_void_p(dadd.ptr), C.c_int64(ld), C.c_void_p(dsum.ptr), C.c_int64(ld), None), "rows_add")
    dev.synchronize()
    assert dev.kernel_error() == 0
    single = dev.mul_mat(w, x)
    got = dst.download(np.float32, n * m).reshape(m, n)
    assert bits_equal(got, single)
    want_sum = single + add[:, :n]
    assert bits_equal(dsum.download(np.float32, ld * m).reshape(m, ld)[:, :n], want_sum)
    # in place: the sum lands on the addend
    dev.check(dev.lib.b200_mul_mat_q8_rows_add(ty, C.c_int64(n), C.c_int64(k), C.c_int64(m), C.c_void_p(w.ptr), C.c_void_p(act.ptr), kind, C.c_void_p(dst.ptr),
                                               C.c_int64(n), C.c_void_p(dadd.ptr), C.c_int64(ld), C.c_void_p(dadd.ptr), C.c_int64(ld), None), "rows_add in place")
    dev.synchronize()
    back = dadd.download(np.float32, ld * m).reshape(m, ld)
    assert bits_equal(back[:, :n], want_sum) and bits_equal(back[:, n:], add[:, n:])


def test_rows_add_refuses_other_shapes(dev):
    assert dev.lib.b200_mul_mat_q8_rows_add_fusable(orc.Q4_K, C.c_int64(4096), C.c_int64(64)) == 0
    assert dev.lib.b200_mul_mat_q8_rows_add_fusable(orc.Q4_K, C.c_int64(4096), C.c_int64(1)) == 0
    assert dev.lib.b200_mul_mat_q8_rows_add_fusable(orc.Q8_0, C.c_int64(4096), C.c_int64(16)) == 0
    one = C.c_void_p(256)
    rc = dev.lib.b200_mul_mat_q8_rows_add(orc.Q4_K, C.c_int64(4096), C.c_int64(4096), C.c_int64(64), one, one, dev.ACT_Q8_K_MIXED, one, C.c_int64(4096), one,
                                          C.c_int64(4096), one, C.c_int64(4096), None)
    assert rc != 0 and b"few-rows kernel" in dev.lib.b200_last_error()
