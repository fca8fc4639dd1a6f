"""The one-token step as ONE persistent kernel (csrc/decode_persistent.cu) against the node-by-node path of the same
numerics policy (fast): the mat-muls keep the CPU routes' accumulation order and attention runs the same unit of work,
so logits and the nodes the kernel materializes are compared bit for bit; the node-by-node fast path is itself held
to the CPU oracle elsewhere (test_gpu_llama.py in exact mode, test_gpu_flash_attn_fast.py for the attention distance).
"""
import importlib
import os

import numpy as np
import pytest

import b200
import orc
from conftest import bits_equal

pytestmark = pytest.mark.gpu

# ragged unit counts on purpose: n_ff = 2816 is 11 groups of 256 (Q4_K units of 8 + 3 groups, Q6_K units of 4 + 4 + 3)
MODEL = dict(n_vocab=1024, n_embd=1024, n_head=8, n_head_kv=2, n_embd_head=128, n_ff=2816, n_layer=3, n_ctx_train=8192,
             rope_mode=0, norm_rms_eps=1e-5, rope_freq_base=500000.0, rope_freq_scale=1.0)
WIDE = dict(MODEL, n_embd=2048, n_head=16, n_head_kv=4, n_ff=5632, n_vocab=4096, n_layer=2)


@pytest.fixture(scope="module")
def ll():
    b200.load()
    return importlib.import_module("llama_rust_b200.llama")


@pytest.fixture
def fast(monkeypatch):
    """fast numerics, with the node-by-node path's attention on the CUDA-core kernel: the unit of work the persistent
    kernel carries (the tensor-core decode kernel, the node path's default, rounds q and p to f16 and differs in bits)"""
    m = b200.load()
    before = m.get_numerics()
    m.set_numerics(m.FAST)
    monkeypatch.setenv("B200_FA_DECODE_MMA", "0")
    yield m
    m.set_numerics(before)


def make_tensors(ll, hp, seed):
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, (ne0, ne1) in ll.tensor_shapes(hp).items():
        ty = ll.q4_k_m_type(name, hp["n_layer"])
        if ty == orc.F32:
            arr = (1.0 + 0.1 * rng.standard_normal(ne0)).astype(np.float32)
        else:
            arr = orc.quantize_rows(ty, (rng.standard_normal((ne1, ne0)) * 0.05).astype(np.float32))
        tensors[name] = (ty, arr, ne0, ne1)
    return tensors


def instance(ll, hp, tensors, n_ctx, persistent):
    old = os.environ.get("B200_DECODE_PERSISTENT")
    os.environ["B200_DECODE_PERSISTENT"] = "1" if persistent else "0"   # read when the backend is created
    try:
        gpu = ll.Llama(hp, n_ctx, 256, cpu_threads=8)
    finally:
        if old is None:
            del os.environ["B200_DECODE_PERSISTENT"]
        else:
            os.environ["B200_DECODE_PERSISTENT"] = old
    for name, (ty, arr, ne0, ne1) in tensors.items():
        gpu.set_tensor(name, ty, arr, ne0, ne1)
    return gpu


NODES = lambda hp: [("Qcur_rope", hp["n_head"] * 128), ("kqv_out", hp["n_head"] * 128), ("ffn_inp", hp["n_embd"]),
                    ("ffn_gate_par", hp["n_ff"]), ("l_out", hp["n_embd"]), ("result_norm", hp["n_embd"])]


def compare_runs(ll, m, hp, seed, prompt_len, n_gen, n_ctx=1024):
    tensors = make_tensors(ll, hp, seed)
    a = instance(ll, hp, tensors, n_ctx, True)
    b = instance(ll, hp, tensors, n_ctx, False)
    rng = np.random.default_rng(seed + 1)
    prompt = rng.integers(0, hp["n_vocab"], prompt_len).astype(np.int32)
    pos = np.arange(prompt_len, dtype=np.int32)
    la, tok = a.decode(prompt, pos, logits=True, argmax=True)
    lb = b.decode(prompt, pos)
    assert bits_equal(la, lb)
    for step in range(n_gen):
        p = prompt_len + step
        before = m.lib.b200_debug_decode_step_launches()
        la, ta = a.decode([tok], [p], logits=True, argmax=True)
        assert m.lib.b200_debug_decode_step_launches() == before + 1, "the step did not take the persistent kernel"
        lb, tb = b.decode([tok], [p], logits=True, argmax=True)
        assert m.lib.b200_debug_decode_step_launches() == before + 1, "the reference instance took the persistent kernel"
        assert m.kernel_error() == 0
        for name, count in NODES(hp):
            na, nb = a.read_node(name, count), b.read_node(name, count)
            assert bits_equal(na, nb), f"step {step}: node {name} differs, max |d| = {np.abs(na - nb).max()}"
        assert bits_equal(la, lb), f"step {step}: logits differ, max |d| = {np.abs(la - lb).max()}"
        assert ta == tb
        tok = ta
    assert a.kv_used() == b.kv_used() == prompt_len + n_gen
    a.close()
    b.close()


def test_persistent_step_equals_node_by_node(ll, fast):
    compare_runs(ll, fast, MODEL, seed=21, prompt_len=7, n_gen=6)


def test_persistent_step_from_an_empty_cache(ll, fast):
    compare_runs(ll, fast, MODEL, seed=22, prompt_len=1, n_gen=3)


def test_persistent_step_crossing_a_256_cell_boundary(ll, fast):
    # the padded cache length grows from 256 to 512 during generation: a new node list, a new phase list
    compare_runs(ll, fast, MODEL, seed=23, prompt_len=252, n_gen=8)


def test_persistent_step_wider_model(ll, fast):
    compare_runs(ll, fast, WIDE, seed=24, prompt_len=40, n_gen=4)


def test_grid_barrier_wait_expiry_returns_with_a_code(ll, fast):
    """One CTA of the persistent step never arrives at a grid barrier (test hook): every other CTA's bounded wait runs
    out, the kernel returns, b200_kernel_error reports code 5, and after a cache reset the same driver gives the same
    bits as the node-by-node path again."""
    tensors = make_tensors(ll, MODEL, 31)
    a = instance(ll, MODEL, tensors, 512, True)
    b = instance(ll, MODEL, tensors, 512, False)
    prompt = np.arange(1, 6, dtype=np.int32)
    pos = np.arange(5, dtype=np.int32)
    tok = a.decode(prompt, pos, logits=False, argmax=True)
    fast.lib.b200_debug_decode_step_wait(4000, 3, 7)   # CTA 3 skips its 8th barrier: the second layer's attention
    try:
        # the decode call reads the device's error word after the step and fails with it: 5 = a grid-barrier wait ran
        # out, 6 = a producer found its ring full for too long (its consumers were stuck at that barrier), 7 = a consumer
        # gave up waiting for a copy; which of the waits that ran out wrote last is a race
        with pytest.raises(b200.load().B200Error, match=r"error code [567]"):
            a.decode([tok], [5])
    finally:
        fast.lib.b200_debug_decode_step_wait(0, -1, -1)
    assert fast.kernel_error() == 0   # the failed call consumed the code
    for gpu in (a, b):
        gpu.kv_clear()
    la, ta = a.decode(prompt, pos, logits=True, argmax=True)
    lb, tb = b.decode(prompt, pos, logits=True, argmax=True)
    assert bits_equal(la, lb) and ta == tb
    before = fast.lib.b200_debug_decode_step_launches()
    la = a.decode([ta], [5])
    lb = b.decode([tb], [5])
    assert fast.lib.b200_debug_decode_step_launches() == before + 1
    assert fast.kernel_error() == 0
    assert bits_equal(la, lb)
    a.close()
    b.close()
