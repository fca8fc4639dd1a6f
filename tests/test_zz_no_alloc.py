"""b200_mul_mat_static_scratch, the MUL_MAT entry point for hosts that cannot allocate.

Some callers of this library may not call cudaMalloc while they run: a decode loop
whose device-memory budget was fixed at start-up, a process whose allocations all go
through its own memory manager.  For them the library offers a MUL_MAT whose
activation scratch is a fixed array inside the loaded module.  The tests drive it
through the C ABI:

* twice in a row on different activations in this process (the array is shared and
  keeps the previous call's contents, so the second call would expose stale state),
  against b200_mul_mat's bits;
* in a fresh child process where it is the FIRST compute call the library sees, so
  that nothing another entry point allocated earlier can hide an allocation of its
  own: the library's allocation counter must stay at zero, the device's free memory
  must not move across the calls, and every result must equal the CPU oracle's bit
  for bit.  The child covers the decode kernel (1 and 3 rows), the mma.sync kernel
  (8 and 12 rows), the integer tcgen05 kernel (40 rows) and a shape for which
  b200_mul_mat would take the two-pass kernel with its extra scratch block (192 rows
  against 4096 weight rows), plus Q6_K, Q8_0 and MXFP4.

The file is named so that pytest collects it last.
"""
import json
import os
import subprocess
import sys

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


# (type, n, k, m): every kernel family the entry point can reach; all fit the 256 KiB array
CHILD_CASES = [
    ("Q4_K", 512, 2048, 1), ("Q4_K", 512, 2048, 3), ("Q4_K", 4096, 4096, 1), ("Q4_K", 256, 1024, 8), ("Q4_K", 256, 1024, 12),
    ("Q4_K", 256, 1024, 40), ("Q4_K", 4096, 1024, 192), ("Q6_K", 256, 1024, 1), ("Q6_K", 256, 1024, 9),
    ("Q8_0", 256, 1024, 2), ("MXFP4", 768, 2048, 5),
]

CHILD = r"""
import ctypes, json, sys
import numpy as np
import b200, orc, synth
dev = b200.load()
dev.set_device(0)
lib = dev.lib

def free_bytes():
    f, t = ctypes.c_size_t(), ctypes.c_size_t()
    dev.check(lib.b200_device_info(0, None, 0, ctypes.byref(f), ctypes.byref(t), None, None, None), "device_info")
    return f.value

cases = json.loads(sys.argv[1])
names = {"Q4_K": orc.Q4_K, "Q6_K": orc.Q6_K, "Q8_0": orc.Q8_0, "MXFP4": orc.MXFP4}
# everything the caller owns is allocated first: weights, activations, results
prepared = []
for name, n, k, m in cases:
    ty = names[name]
    W = synth.weights(ty, n, k, seed=61)
    x = synth.activations(m, k, seed=62 + m)
    prepared.append((name, ty, n, k, m, W, x, dev.Weight(ty, W, k), dev.device_array(x), dev.DeviceBuffer(4 * m * n)))
dev.synchronize()
report = {"alloc_before": int(lib.b200_debug_alloc_count()), "free_before": free_bytes(), "cases": []}
for rep in range(2):   # two passes: the second sees whatever the first left in the array
    for name, ty, n, k, m, W, x, w, dx, out in prepared:
        rc = lib.b200_mul_mat_static_scratch(ty, n, k, m, w.ptr, dx.ptr, k, out.ptr, n, 0, None)
        if rc != 0:
            report["cases"].append({"case": [name, n, k, m], "rc": rc, "error": lib.b200_last_error().decode()})
            continue
        got = out.download(np.float32, m * n).reshape(m, n)
        want, _ = orc.mul_mat(ty, W, x)
        report["cases"].append({"case": [name, n, k, m], "rc": 0, "pass": rep,
                                "bit_exact": bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))})
dev.synchronize()
report["alloc_after"] = int(lib.b200_debug_alloc_count())
report["free_after"] = free_bytes()
report["kernel_error"] = dev.kernel_error()
print("REPORT " + json.dumps(report))
"""


def test_static_scratch_first_call_in_a_fresh_process_allocates_nothing():
    here = os.path.dirname(os.path.abspath(__file__))
    # eager module loading: with lazy loading the first launch of each kernel maps its code, which moves the
    # device's free-memory figure for reasons that have nothing to do with the entry point
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER", PYTHONPATH=here + os.pathsep + os.environ.get("PYTHONPATH", ""))
    for var in ("B200_GEMM_TCGEN05_F16", "B200_GEMV_KSPLIT"):
        env.pop(var, None)
    r = subprocess.run([sys.executable, "-c", CHILD, json.dumps(CHILD_CASES)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("REPORT ")][-1]
    rep = json.loads(line[len("REPORT "):])
    assert len(rep["cases"]) == 2 * len(CHILD_CASES)
    for c in rep["cases"]:
        assert c["rc"] == 0, c
        assert c["bit_exact"], c
    assert rep["kernel_error"] == 0
    assert rep["alloc_before"] == 0 and rep["alloc_after"] == 0, rep
    assert rep["free_after"] == rep["free_before"], rep
