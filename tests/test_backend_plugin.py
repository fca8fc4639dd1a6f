"""The ggml backend plug-in face of the library, driven like the reference's registry and scheduler
drive a dlopen-ed backend (crates/ggml/src/backend.rs:2454-2559 loads a stub .so the same way;
backend_sched.rs:2357-2459 runs a two-backend split against a mock device)."""
import ctypes as C

import numpy as np
import pytest

import b200
import ggml_plugin as gp
import orc
import synth
from conftest import bits_equal


def lib_path():
    return b200.load().LIB_PATH


def test_registry_entry_points_without_a_gpu():
    """dlopen, ggml_backend_init, api_version 2, name; with no usable device the score is 0 and the
    registry enumerates nothing (the reference then leaves the backend unregistered)."""
    lib, reg = gp.load_backend(lib_path())
    r = reg.contents
    assert r.api_version == 2
    assert r.iface.get_name(C.cast(reg, C.c_void_p)) == b"B200"
    n = r.iface.get_device_count(C.cast(reg, C.c_void_p))
    score = lib.ggml_backend_score()
    assert (score == 0) == (n == 0)
    assert r.iface.get_proc_address(C.cast(reg, C.c_void_p), b"b200_backend_set_cpu_threads")
    assert not r.iface.get_proc_address(C.cast(reg, C.c_void_p), b"no_such_symbol")
    assert not r.iface.get_device(C.cast(reg, C.c_void_p), 10 ** 6)


@pytest.fixture(scope="module")
def sess():
    lib, reg = gp.load_backend(lib_path())
    if reg.contents.iface.get_device_count(C.cast(reg, C.c_void_p)) == 0:
        pytest.fail("no B200 device enumerated")
    s = gp.Session(lib, reg, params=b"cpu_threads=8")
    yield s
    s.close()


@pytest.mark.gpu
def test_device_and_buffer_type(sess):
    d = sess.dev
    assert d.iface.get_type(sess.devp) == 1  # GPU
    assert d.iface.get_name(sess.devp).startswith(b"B200")
    assert b"B200" in d.iface.get_description(sess.devp)
    free, total = C.c_size_t(), C.c_size_t()
    d.iface.get_memory(sess.devp, C.byref(free), C.byref(total))
    assert 0 < free.value <= total.value
    props = gp.DevProps()
    d.iface.get_props(sess.devp, C.byref(props))
    assert props.type == 1 and props.memory_total == total.value
    assert d.iface.supports_buft(sess.devp, sess.buftp)
    assert not sess.buft.iface.is_host(sess.buftp)
    assert sess.buft.iface.get_alignment(sess.buftp) % 32 == 0  # ggml's tensor alignment is 32
    assert sess.be.iface.get_name(sess.bep).startswith(b"B200")


@pytest.mark.gpu
def test_buffer_round_trips(sess):
    x = np.arange(1000, dtype=np.float32)
    t = sess.new_tensor(gp.F32, [1000])
    sess.set(t, x)
    assert np.array_equal(sess.get(t, np.float32, 1000), x)
    sess.buf.iface.memset_tensor(sess.bufp, C.byref(t), 0, 0, 4000)
    assert not sess.get(t, np.float32, 1000).any()
    # a quantized tensor is re-ordered on the way in and restored on the way out; 40 rows pad to 64
    W = synth.weights(orc.Q4_K, 40, 512, seed=1)
    tw = sess.new_tensor(orc.Q4_K, [512, 40])
    assert sess.buft.iface.get_alloc_size(sess.buftp, C.byref(tw)) == 2 * 2 * 4608
    sess.set(tw, W)
    assert np.array_equal(sess.get(tw, np.uint8, W.size), W.ravel())


@pytest.mark.gpu
def test_supports_op_accepts_the_hot_path_and_nothing_else(sess):
    w = sess.new_tensor(orc.Q4_K, [512, 64])
    x = sess.new_tensor(gp.F32, [512, 3])
    d = sess.new_tensor(gp.F32, [64, 3])
    d.op = gp.OP_MUL_MAT
    d.src[0], d.src[1] = C.pointer(w), C.pointer(x)
    assert sess.supports(d)
    wf = sess.new_tensor(gp.F32, [512, 64])
    d.src[0] = C.pointer(wf)
    assert not sess.supports(d)          # F32 weights are not on this path
    d.src[0] = C.pointer(w)
    d.op = gp.OP_ADD
    assert not sess.supports(d)          # another backend (the CPU one) takes it
    v = sess.new_tensor(gp.F32, [64, 3], alloc=False)
    v.op = gp.OP_VIEW
    assert sess.supports(v)


@pytest.mark.gpu
@pytest.mark.parametrize("ty", [orc.Q4_K, orc.Q6_K, orc.Q8_0, orc.MXFP4], ids=lambda t: orc.TYPE_NAMES[t])
def test_graph_compute_mul_mat(sess, ty):
    n, k, m = 256, 1024, 5
    W, X = synth.weights(ty, n, k, seed=2), synth.activations(m, k, seed=3)
    w = sess.new_tensor(ty, [k, n], b"w")
    x = sess.new_tensor(gp.F32, [k, m], b"x")
    d = sess.new_tensor(gp.F32, [n, m], b"dst")
    d.op = gp.OP_MUL_MAT
    d.src[0], d.src[1] = C.pointer(w), C.pointer(x)
    sess.set(w, W)
    sess.set(x, X)
    assert sess.compute([d]) == 0, sess.last_error()
    want, _ = orc.mul_mat(ty, W, X)
    assert bits_equal(sess.get(d, np.float32, n * m).reshape(m, n), want)


@pytest.mark.gpu
def test_graph_compute_mul_mat_id_and_flash_attn(sess):
    E, n, k, n_tok, top = 4, 64, 512, 6, 2
    W = synth.weights(orc.MXFP4, E * n, k, seed=4).reshape(E, n, -1)
    B = synth.activations(n_tok * top, k, seed=5).reshape(n_tok, top, k)
    ids = np.stack([np.random.default_rng(i).permutation(E)[:top] for i in range(n_tok)]).astype(np.int32)
    tw = sess.new_tensor(orc.MXFP4, [k, n, E])
    tb = sess.new_tensor(gp.F32, [k, top, n_tok])
    ti = sess.new_tensor(gp.I32, [top, n_tok])
    td = sess.new_tensor(gp.F32, [n, top, n_tok])
    td.op = gp.OP_MUL_MAT_ID
    td.src[0], td.src[1], td.src[2] = C.pointer(tw), C.pointer(tb), C.pointer(ti)
    sess.set(tw, W)
    sess.set(tb, B)
    sess.set(ti, ids)
    # attention over a KV-cache-shaped view: rows of [h_kv * d] per position
    H, Hkv, D, T, n_kv = 8, 2, 64, 1, 600
    rng = np.random.default_rng(6)
    q = rng.standard_normal((H, T, D)).astype(np.float32)
    kk = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    vv = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    tq = sess.new_tensor(gp.F32, [D, T, H])
    tk = sess.new_tensor(gp.F16, [D * Hkv, n_kv])
    tv = sess.new_tensor(gp.F16, [D * Hkv, n_kv])
    sess.set(tq, q)
    sess.set(tk, np.ascontiguousarray(np.transpose(kk, (1, 0, 2))))
    sess.set(tv, np.ascontiguousarray(np.transpose(vv, (1, 0, 2))))
    kview, vview = gp.Tensor(), gp.Tensor()
    for view, src in ((kview, tk), (vview, tv)):
        view.type, view.buffer, view.data = gp.F16, src.buffer, src.data
        view.ne[0], view.ne[1], view.ne[2], view.ne[3] = D, n_kv, Hkv, 1
        view.nb[0], view.nb[1], view.nb[2], view.nb[3] = 2, D * Hkv * 2, D * 2, D * Hkv * 2 * n_kv
        view.view_src = C.pointer(src)
    to = sess.new_tensor(gp.F32, [D, H, T])
    to.op = gp.OP_FLASH_ATTN_EXT
    to.src[0], to.src[1], to.src[2] = C.pointer(tq), C.pointer(kview), C.pointer(vview)
    C.memmove(C.addressof(to.op_params), np.array([0.125, 0.0, 0.0], dtype=np.float32).ctypes.data, 12)
    assert sess.compute([td, to]) == 0, sess.last_error()
    want, _ = orc.mul_mat_id(orc.MXFP4, W, B, ids)
    assert bits_equal(sess.get(td, np.float32, n_tok * top * n).reshape(n_tok, top, n), want)
    fa, path = orc.flash_attn(q, kk, vv, None, 0.125, n_chunks=8)
    assert path == orc.FA_SPLIT_KV
    assert bits_equal(sess.get(to, np.float32, T * H * D).reshape(T, H, D), fa)


@pytest.mark.gpu
def test_graph_compute_refuses_with_a_status(sess):
    a = sess.new_tensor(gp.F32, [8])
    a.op = gp.OP_ADD
    assert sess.compute([a]) == 3      # GGML_STATUS_BACKEND_ERROR, no abort
    assert "not supported" in sess.last_error()
