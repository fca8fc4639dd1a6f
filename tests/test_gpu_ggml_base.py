"""The libggml-base-shaped export set driven the way the reference's ForeignExecutor drives a foreign ggml
(crates/ggml/src/backend_emit.rs:439-572 new, :895-1042 graph_compute): devices by type, scheduler over
[gpu, cpu], weights in device and host buffers, a per-step context whose tensors get op / src / op_params
written directly, alloc_graph -> tensor_set -> graph_compute -> tensor_get -> reset.  Results against the
CPU oracle, bit for bit."""
import ctypes as C
import struct

import numpy as np
import pytest

import b200
import ggml_base
import orc
import orc_glue
import synth
from conftest import bits_equal
from ggml_plugin import F32

pytestmark = pytest.mark.gpu

OP_RMS_NORM, OP_MUL, OP_MUL_MAT, OP_SOFT_MAX = 25, 7, 29, 46
EPS = 1e-5


@pytest.fixture(scope="module")
def ex():
    """what ForeignExecutor::new holds"""
    b200.load()
    lib = ggml_base.load()
    lib.ggml_backend_load_all_from_path(b".")
    cpu_dev, gpu_dev = lib.ggml_backend_dev_by_type(0), lib.ggml_backend_dev_by_type(1)
    assert cpu_dev and gpu_dev, "no GPU device registered"
    assert lib.ggml_backend_dev_by_name(lib.ggml_backend_dev_name(gpu_dev)) == gpu_dev
    cpu_be, gpu_be = lib.ggml_backend_dev_init(cpu_dev, None), lib.ggml_backend_dev_init(gpu_dev, None)
    set_n = lib.ggml_backend_reg_get_proc_address(lib.ggml_backend_dev_backend_reg(cpu_dev), b"ggml_backend_set_n_threads")
    C.CFUNCTYPE(None, C.c_void_p, C.c_int)(set_n)(cpu_be, 8)
    backends = (C.c_void_p * 2)(gpu_be, cpu_be)
    sched = lib.ggml_backend_sched_new(backends, None, 2, 2048, False, True)
    assert sched
    model_ctx = lib.ggml_init(ggml_base.InitParams(lib.ggml_tensor_overhead() * 64, None, True))
    yield dict(lib=lib, cpu_dev=cpu_dev, gpu_dev=gpu_dev, cpu_be=cpu_be, gpu_be=gpu_be, sched=sched, model_ctx=model_ctx, keep=[])
    lib.ggml_backend_sched_free(sched)
    lib.ggml_free(model_ctx)
    lib.ggml_backend_free(gpu_be)
    lib.ggml_backend_free(cpu_be)


def device_weight(ex, ty, blocks, ne, name):
    lib = ex["lib"]
    t = ggml_base.new_tensor(lib, ex["model_ctx"], ty, ne, name)
    buft = lib.ggml_backend_dev_buffer_type(ex["gpu_dev"])
    buf = lib.ggml_backend_buft_alloc_buffer(buft, lib.ggml_backend_buft_get_alloc_size(buft, t) + lib.ggml_backend_buft_get_alignment(buft))
    assert buf
    lib.ggml_backend_buffer_set_usage(buf, 1)
    assert lib.ggml_backend_tensor_alloc(buf, t, lib.ggml_backend_buffer_get_base(buf)) == 0
    blocks = np.ascontiguousarray(blocks)
    lib.ggml_backend_tensor_set(t, blocks.ctypes.data, 0, blocks.nbytes)
    ex["keep"].append(buf)
    return t


def host_weight(ex, arr, ne, name):
    """a weight a partial -ngl placement left on the CPU side: a host buffer wrapped around the caller's memory"""
    lib = ex["lib"]
    t = ggml_base.new_tensor(lib, ex["model_ctx"], F32, ne, name)
    buf = lib.ggml_backend_cpu_buffer_from_ptr(arr.ctypes.data, arr.nbytes)
    lib.ggml_backend_buffer_set_usage(buf, 1)
    assert lib.ggml_backend_tensor_alloc(buf, t, arr.ctypes.data) == 0
    ex["keep"] += [buf, arr]
    return t


def test_executor_flow_norm_mul_matmul(ex):
    lib, sched = ex["lib"], ex["sched"]
    k, n = 512, 64
    W = synth.weights(orc.Q4_K, n, k, seed=81)
    norm_w = (1.0 + 0.1 * np.random.default_rng(82).standard_normal(k)).astype(np.float32)
    wq = device_weight(ex, orc.Q4_K, W, [k, n], b"blk.0.attn_q.weight")
    wn = host_weight(ex, norm_w, [k], b"blk.0.attn_norm.weight")
    assert lib.ggml_backend_sched_get_n_backends(sched) == 2 and lib.ggml_backend_sched_get_backend(sched, 0) == ex["gpu_be"]
    for step, m in enumerate((3, 1, 3)):
        size = 64
        ctx = lib.ggml_init(ggml_base.InitParams(lib.ggml_tensor_overhead() * 16 + lib.ggml_graph_overhead_custom(size, False), None, True))
        x = ggml_base.new_tensor(lib, ctx, F32, [k, m], b"inp")
        norm = ggml_base.op_node(lib, ctx, F32, [k, m], OP_RMS_NORM, [x], b"norm", struct.pack("<f", EPS))
        mul = ggml_base.op_node(lib, ctx, F32, [k, m], OP_MUL, [norm, wn], b"attn_norm")
        q = ggml_base.op_node(lib, ctx, F32, [n, m], OP_MUL_MAT, [wq, mul], b"Qcur")
        lib.ggml_set_input(x)
        lib.ggml_set_output(q)
        g = lib.ggml_new_graph_custom(ctx, size, False)
        lib.ggml_build_forward_expand(g, q)
        assert lib.ggml_graph_n_nodes(g) == 3
        assert lib.ggml_backend_sched_alloc_graph(sched, g)
        xs = synth.activations(m, k, seed=90 + step)
        lib.ggml_backend_tensor_set(x, xs.ctypes.data, 0, xs.nbytes)
        assert lib.ggml_backend_sched_graph_compute(sched, g) == 0
        lib.ggml_backend_sched_synchronize(sched)
        got = np.empty((m, n), dtype=np.float32)
        lib.ggml_backend_tensor_get(q, got.ctypes.data, 0, got.nbytes)
        normed = orc_glue.mul(orc_glue.rms_norm(xs, EPS), np.tile(norm_w, (m, 1)))
        want, _ = orc.mul_mat(orc.Q4_K, W, normed)
        assert bits_equal(got, want), f"step {step}: max |d| = {np.abs(got - want).max()}"
        # an intermediate is readable too, and nodes report the device backend, host leaves the CPU one
        mid = np.empty((m, k), dtype=np.float32)
        lib.ggml_backend_tensor_get(mul, mid.ctypes.data, 0, mid.nbytes)
        assert bits_equal(mid, normed)
        assert lib.ggml_backend_sched_get_tensor_backend(sched, q) == ex["gpu_be"]
        assert lib.ggml_backend_sched_get_tensor_backend(sched, wn) == ex["cpu_be"]
        assert lib.ggml_backend_sched_get_buffer_size(sched, ex["gpu_be"]) > 0
        lib.ggml_backend_sched_reset(sched)
        lib.ggml_free(ctx)


def test_unsupported_node_is_refused_at_alloc(ex):
    lib, sched = ex["lib"], ex["sched"]
    ctx = lib.ggml_init(ggml_base.InitParams(lib.ggml_tensor_overhead() * 8 + lib.ggml_graph_overhead_custom(16, False), None, True))
    x = ggml_base.new_tensor(lib, ctx, F32, [64, 2], b"x")
    sm = ggml_base.op_node(lib, ctx, F32, [64, 2], OP_SOFT_MAX, [x], b"soft")
    g = lib.ggml_new_graph_custom(ctx, 16, False)
    lib.ggml_build_forward_expand(g, sm)
    assert not lib.ggml_backend_sched_alloc_graph(sched, g), "no CPU compute path: the graph has to be refused, not half-run"
    lib.ggml_backend_sched_reset(sched)
    lib.ggml_free(ctx)
