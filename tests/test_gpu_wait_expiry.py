"""A bounded wait that runs out: the kernel returns, reports a code, and the device stays usable.

Every wait inside the library's kernels has a poll limit.  This test makes one run out without faulting or
hanging anything: through the library's test hook the streaming decode kernel gets a short poll limit and a
producer that leaves the first ring unit of every CTA unfilled, so the consumers of that unit give up.  The
launch must return, b200_kernel_error must report code 1 (producer gave up) or 2 (a consumer did), no output
row may have been written (a row tile's results are stored only after all of its K groups arrived), and the
next normal launch must be bit-exact with the CPU oracle.
"""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu


def test_streaming_kernel_wait_expiry_reports_a_code_and_the_next_launch_is_exact():
    dev = b200.load()
    assert dev.device_count() > 0
    dev.set_device(0)
    n, k = 4096, 4096   # 128 row tiles: the streaming kernel, one tile (two ring units) per CTA
    W = synth.weights(orc.Q4_K, n, k, seed=71, period=512)
    w = dev.Weight(orc.Q4_K, W, k)
    x = synth.activations(1, k, seed=72)
    dx = dev.device_array(x)
    out = dev.DeviceBuffer(4 * n)
    want, _ = orc.mul_mat(orc.Q4_K, W, x)

    dev.lib.b200_debug_stream_wait(1 << 20, -1)   # the streaming kernel with its normal poll limit, nothing skipped
    try:
        dev.mul_mat_device(w, dx, 1, out)         # a normal launch first: the kernel works
        dev.synchronize()
    finally:
        dev.lib.b200_debug_stream_wait(0, -1)
    assert dev.kernel_error() == 0
    assert bits_equal(out.download(np.float32, n), want.ravel())

    dev.check(dev.lib.b200_memset(out.ptr, 0xFF, 4 * n, None), "memset")
    dev.synchronize()
    dev.lib.b200_debug_stream_wait(2000, 0)
    try:
        dev.mul_mat_device(w, dx, 1, out)
        dev.synchronize()           # returns: the waits gave up after 2000 polls
    finally:
        dev.lib.b200_debug_stream_wait(0, -1)
    assert dev.kernel_error() in (1, 2)
    assert dev.kernel_error() == 0   # the read cleared it
    assert (out.download(np.uint32, n) == 0xFFFFFFFF).all(), "an aborted row tile must not store results"

    dev.lib.b200_debug_stream_wait(1 << 20, -1)
    try:
        dev.mul_mat_device(w, dx, 1, out)         # the same kernel again, undisturbed
        dev.synchronize()
    finally:
        dev.lib.b200_debug_stream_wait(0, -1)
    assert dev.kernel_error() == 0
    assert bits_equal(out.download(np.float32, n), want.ravel())


def test_second_device_in_the_same_process():
    """Kernels that need more than 48 KB of dynamic shared memory set a per-(function, device) attribute: after
    device 0 has run them, device 1 must get its own."""
    dev = b200.load()
    if dev.device_count() < 2:
        pytest.skip("needs two devices")
    cases = [(orc.Q4_K, 256, 4096, 3), (orc.Q6_K, 256, 4096, 1), (orc.Q4_K, 256, 2048, 16)]
    try:
        for d in (0, 1):
            dev.set_device(d)
            for ty, n, k, m in cases:
                W = synth.weights(ty, n, k, seed=81)
                x = synth.activations(m, k, seed=82)
                want, _ = orc.mul_mat(ty, W, x)
                assert bits_equal(dev.mul_mat(dev.Weight(ty, W, k), x), want), (d, ty, m)
            assert dev.kernel_error() == 0
    finally:
        dev.set_device(0)


def test_fast_prompt_mat_mul_partial_tile_wait_expiry(monkeypatch):
    """The fast-numerics prompt mat-mul cuts its work into one run per CTA; a tile cut between two CTAs is finished by the
    one holding its first half, which waits (bounded) for the other's partial tile.  Here CTA 1 never announces its half:
    the wait of CTA 0 runs out after 2000 polls, the kernel returns, b200_kernel_error reports code 4, tile 0 is left
    unwritten, every other tile is what an undisturbed launch gives, and the next launch is undisturbed."""
    dev = b200.load()
    dev.set_device(0)
    n, k, m = 4096, 4096, 512
    monkeypatch.setenv("B200_GEMM_FAST_CTAS", "128")   # 64 tiles of 128 x 256, sixteen super-blocks each: every tile in two halves
    W = synth.weights(orc.Q4_K, n, k, seed=81, period=512)
    w = dev.Weight(orc.Q4_K, W, k)
    x = synth.activations(m, k, seed=82)
    dx = dev.device_array(x)
    out = dev.DeviceBuffer(4 * n * m)
    dev.set_numerics(dev.FAST)
    try:
        dev.mul_mat_device(w, dx, m, out)
        dev.synchronize()
        assert dev.kernel_error() == 0
        good = out.download(np.float32, n * m).reshape(m, n).copy()

        dev.check(dev.lib.b200_memset(out.ptr, 0xFF, 4 * n * m, None), "memset")
        dev.synchronize()
        dev.lib.b200_debug_gemm_fast_wait(2000, 1)
        try:
            dev.mul_mat_device(w, dx, m, out)
            dev.synchronize()           # returns: the wait gave up
        finally:
            dev.lib.b200_debug_gemm_fast_wait(0, -1)
        assert dev.kernel_error() == 4
        assert dev.kernel_error() == 0   # the read cleared it (and lowered the flags)
        got = out.download(np.uint32, n * m).reshape(m, n)
        assert (got[:256, :128] == 0xFFFFFFFF).all(), "the unfinished tile must not be stored"
        rest = np.ones((m, n), dtype=bool)
        rest[:256, :128] = False
        assert (got[rest] == good.view(np.uint32)[rest]).all()

        dev.mul_mat_device(w, dx, m, out)
        dev.synchronize()
        assert dev.kernel_error() == 0
        assert bits_equal(out.download(np.float32, n * m).reshape(m, n), good)
    finally:
        dev.set_numerics(dev.EXACT)


def test_few_rows_ring_mat_mul_wait_expiry():
    """The persistent few-rows mat-mul (8 to 31 activation rows) passes ring slots from a producer warp to multiply warps to
    chain warps.  Here the producer of the first CTA never fills its sixth unit: the multiply warp's wait runs out after
    20000 polls, the CTA winds down without storing, the kernel returns, b200_kernel_error reports code 4, that CTA's row
    tile is left unwritten, every other tile is what an undisturbed launch gives, and the next launch is undisturbed."""
    dev = b200.load()
    dev.set_device(0)
    n, k, m = 4096, 4096, 16   # 128 row tiles: one per CTA
    W = synth.weights(orc.Q4_K, n, k, seed=91, period=512)
    w = dev.Weight(orc.Q4_K, W, k)
    x = synth.activations(m, k, seed=92)
    dx = dev.device_array(x)
    out = dev.DeviceBuffer(4 * n * m)
    dev.mul_mat_device(w, dx, m, out)
    dev.synchronize()
    assert dev.kernel_error() == 0
    good = out.download(np.float32, n * m).reshape(m, n).copy()
    want, _ = orc.mul_mat(orc.Q4_K, W, x)
    assert bits_equal(good, want)

    dev.check(dev.lib.b200_memset(out.ptr, 0xFF, 4 * n * m, None), "memset")
    dev.synchronize()
    dev.lib.b200_debug_rows_ring_wait(20000, 5)
    try:
        dev.mul_mat_device(w, dx, m, out)
        dev.synchronize()           # returns: the wait gave up
    finally:
        dev.lib.b200_debug_rows_ring_wait(0, -1)
    assert dev.kernel_error() == 4
    assert dev.kernel_error() == 0
    got = out.download(np.uint32, n * m).reshape(m, n)
    assert (got[:, :32] == 0xFFFFFFFF).all(), "the unfinished tile must not be stored"
    assert (got[:, 32:] == good.view(np.uint32)[:, 32:]).all()

    dev.mul_mat_device(w, dx, m, out)
    dev.synchronize()
    assert dev.kernel_error() == 0
    assert bits_equal(out.download(np.float32, n * m).reshape(m, n), good)
