"""The libggml-base-shaped export set (include/ggml_base_b200.h) without a GPU: every CLibSyms symbol is
there, contexts and graphs behave like ggml's, the host device serves buffers, the placement rule is the
reference's."""
import ctypes as C
import struct

import numpy as np
import pytest

import ggml_base
from ggml_plugin import F32, OP_ADD, OP_NONE

OP_RMS_NORM, OP_MUL = 25, 7


@pytest.fixture(scope="module")
def lib():
    return ggml_base.load()


def test_every_clibsyms_symbol_resolves(lib):
    assert len(ggml_base.CLIB_SYMS) == 54   # the fields of CLibSyms, the optional copy-callback setter included
    for name in ggml_base.CLIB_SYMS:
        assert getattr(lib, name) is not None, name


def test_context_arena_and_tensor_layout(lib):
    over = lib.ggml_tensor_overhead()
    assert over == 32 + 336
    ctx = lib.ggml_init(ggml_base.InitParams(over * 3, None, True))
    a = ggml_base.new_tensor(lib, ctx, 12, [512, 7], b"w")        # Q4_K: 144 bytes per 256
    assert list(a.contents.ne) == [512, 7, 1, 1] and list(a.contents.nb) == [144, 288, 2016, 2016]
    assert a.contents.name == b"w" and not a.contents.data and a.contents.op == OP_NONE
    b = ggml_base.new_tensor(lib, ctx, F32, [5, 3, 2])
    assert list(b.contents.nb) == [4, 20, 60, 120]
    ggml_base.new_tensor(lib, ctx, F32, [1])
    arr = (C.c_int64 * 1)(1)
    assert not lib.ggml_new_tensor(ctx, F32, 1, arr), "a fourth tensor does not fit: NULL, not an abort"
    assert not lib.ggml_new_tensor(ctx, 12, 1, (C.c_int64 * 1)(100)), "row length not a multiple of the block"
    lib.ggml_free(ctx)


def test_forward_expand_orders_sources_first_and_visits_once(lib):
    size = 64
    ctx = lib.ggml_init(ggml_base.InitParams(lib.ggml_tensor_overhead() * 16 + lib.ggml_graph_overhead_custom(size, False), None, True))
    x = ggml_base.new_tensor(lib, ctx, F32, [8], b"x")
    w = ggml_base.new_tensor(lib, ctx, F32, [8], b"w")
    norm = ggml_base.op_node(lib, ctx, F32, [8], OP_RMS_NORM, [x], b"norm", struct.pack("<f", 1e-5))
    mul = ggml_base.op_node(lib, ctx, F32, [8], OP_MUL, [norm, w], b"mul")
    add = ggml_base.op_node(lib, ctx, F32, [8], OP_ADD, [mul, x])
    side = ggml_base.op_node(lib, ctx, F32, [8], OP_ADD, [norm, norm], b"side")
    g = lib.ggml_new_graph_custom(ctx, size, False)
    lib.ggml_build_forward_expand(g, add)
    lib.ggml_build_forward_expand(g, side)      # a second root: only what is new is appended
    lib.ggml_build_forward_expand(g, mul)       # already there
    assert lib.ggml_graph_n_nodes(g) == 4
    names = [lib.ggml_graph_node(g, i).contents.name for i in range(4)]
    assert names == [b"norm", b"mul", b"node_2", b"side"]
    assert lib.ggml_graph_node(g, -1).contents.name == b"side"
    assert not lib.ggml_graph_node(g, 4)
    assert g.contents.n_leafs == 2
    nodes = lib.ggml_graph_nodes(g)
    assert nodes[1].contents.name == b"mul"
    lib.ggml_set_input(x)
    lib.ggml_set_output(add)
    assert x.contents.flags == 1 and add.contents.flags == 2
    lib.ggml_free(ctx)


def test_host_buffers_round_trip(lib):
    buft = lib.ggml_backend_cpu_buffer_type()
    assert lib.ggml_backend_buft_get_alignment(buft) == 32
    ctx = lib.ggml_init(ggml_base.InitParams(lib.ggml_tensor_overhead() * 4, None, True))
    t = ggml_base.new_tensor(lib, ctx, F32, [16, 4], b"t")
    assert lib.ggml_backend_buft_get_alloc_size(buft, t) == 256
    buf = lib.ggml_backend_buft_alloc_buffer(buft, 1024)
    base = lib.ggml_backend_buffer_get_base(buf)
    assert lib.ggml_backend_tensor_alloc(buf, t, base + 64) == 0
    src = np.arange(64, dtype=np.float32)
    lib.ggml_backend_tensor_set(t, src.ctypes.data, 0, src.nbytes)
    out = np.zeros(16, dtype=np.float32)
    lib.ggml_backend_tensor_get(t, out.ctypes.data, 64, 64)
    assert np.array_equal(out, src[16:32])
    # a view of row 2
    v = ggml_base.new_tensor(lib, ctx, F32, [16], b"v")
    v.contents.view_src = t
    v.contents.view_offs = 128
    assert lib.ggml_backend_view_init(v) == 0
    lib.ggml_backend_tensor_get(v, out.ctypes.data, 0, 64)
    assert np.array_equal(out, src[32:48])
    lib.ggml_backend_buffer_clear(buf, 0)
    lib.ggml_backend_tensor_get(t, out.ctypes.data, 0, 64)
    assert not out.any()
    lib.ggml_backend_buffer_free(buf)
    # memory the caller owns (the reference wraps its mmap'ed weights this way)
    mine = np.full(32, 7.0, dtype=np.float32)
    wrapped = lib.ggml_backend_cpu_buffer_from_ptr(mine.ctypes.data, mine.nbytes)
    assert lib.ggml_backend_buffer_get_base(wrapped) == mine.ctypes.data
    lib.ggml_backend_buffer_free(wrapped)
    assert mine[0] == 7.0
    lib.ggml_free(ctx)


def test_registry_always_has_the_host_device(lib):
    lib.ggml_backend_load_all_from_path(b"/nonexistent")
    n = lib.ggml_backend_dev_count()
    cpu = lib.ggml_backend_dev_by_type(0)
    assert cpu and lib.ggml_backend_dev_name(cpu) == b"CPU"
    assert lib.ggml_backend_dev_get(n - 1) == cpu and not lib.ggml_backend_dev_get(n)
    assert lib.ggml_backend_dev_by_name(b"cpu") == cpu and not lib.ggml_backend_dev_by_name(b"Vulkan0")
    assert lib.ggml_backend_dev_buffer_type(cpu) == lib.ggml_backend_cpu_buffer_type()
    reg = lib.ggml_backend_dev_backend_reg(cpu)
    assert lib.ggml_backend_reg_get_proc_address(reg, b"ggml_backend_set_n_threads")
    assert not lib.ggml_backend_reg_get_proc_address(reg, b"no_such_entry")
    be = lib.ggml_backend_dev_init(cpu, None)
    assert be
    # a scheduler needs a GPU backend: with the host one alone it refuses
    arr = (C.c_void_p * 1)(be)
    assert not lib.ggml_backend_sched_new(arr, None, 1, 2048, False, False)
    lib.ggml_backend_free(be)
    assert lib.ggml_time_us() > 0


def test_ngl_placement_rule(lib):
    # crates/ggml/src/backend_emit.rs:173-190 on a 32-layer model (the output layer counts as layer 32)
    assert lib.b200_gpu_layer_start(32, 0) == 2 ** 64 - 1
    assert lib.b200_gpu_layer_start(32, 33) == 0 and lib.b200_gpu_layer_start(32, 99) == 0
    assert lib.b200_gpu_layer_start(32, 10) == 23
    assert [il for il in range(34) if lib.b200_layer_on_gpu(32, 10, il)] == list(range(23, 33))
    assert not any(lib.b200_layer_on_gpu(32, -1, il) for il in range(34))
