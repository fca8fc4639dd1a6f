"""b200_mul_mat_static_scratch, the MUL_MAT entry point for hosts that cannot allocate.

Some callers of this library may not call cudaMalloc while they run: a decode loop
whose device-memory budget was fixed at start-up, a process whose allocations all go
through its own memory manager.  For them the library offers a MUL_MAT whose
activation scratch is a fixed array inside the loaded module.  This test drives it
through the C ABI twice in a row on different activations (the array is shared and
keeps the previous call's contents, so the second call would expose stale state)
and requires the very same bits as b200_mul_mat, which the other tests check
against the CPU oracle.  It is named so that pytest collects it last.
"""
import numpy as np
import pytest

import b200
import orc
import synth

pytestmark = pytest.mark.gpu


def run(dev, fn, w, x):
    m, k = x.shape
    dx = dev.device_array(x)
    out = dev.DeviceBuffer(4 * m * w.n_rows)
    dev.check(fn(w.ty, w.n_rows, k, m, w.ptr, dx.ptr, k, out.ptr, w.n_rows, 0, None), "mul_mat")
    return out.download(np.float32, m * w.n_rows)


def test_static_scratch_matches_allocating_entry_point_twice():
    dev = b200.load()
    assert dev.device_count() > 0
    dev.set_device(0)
    n, k = 512, 2048
    w = dev.Weight(orc.Q4_K, synth.weights(orc.Q4_K, n, k, seed=21), k)
    for seed, m in ((31, 1), (32, 3)):
        x = synth.activations(m, k, seed=seed)
        want = run(dev, dev.lib.b200_mul_mat, w, x)
        got = run(dev, dev.lib.b200_mul_mat_static_scratch, w, x)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"call with m={m}"


def test_static_scratch_refuses_what_does_not_fit():
    dev = b200.load()
    dev.set_device(0)
    limit = dev.lib.b200_static_scratch_nbytes()
    assert limit == 256 * 1024
    n, k, m = 32, 16384, 20  # 20 x 16384 int8 quants alone exceed the array
    w = dev.Weight(orc.Q4_K, synth.weights(orc.Q4_K, n, k, seed=22), k)
    dx = dev.DeviceBuffer(4 * m * k)
    out = dev.DeviceBuffer(4 * m * n)
    rc = dev.lib.b200_mul_mat_static_scratch(w.ty, n, k, m, w.ptr, dx.ptr, k, out.ptr, n, 0, None)
    assert rc == 3
    assert b"fixed array" in dev.lib.b200_last_error()
