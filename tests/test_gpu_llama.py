"""The Llama decode driver (include/llama_b200.h) against the CPU oracle's Llama forward on small
synthetic models with the Q4_K_M tensor-type mix: prompt batches of every mat-mul / attention route,
then greedy single-token steps.  Logits are compared bit for bit."""
import importlib

import numpy as np
import pytest

import b200
import orc
import orc_glue
from conftest import bits_equal

pytestmark = pytest.mark.gpu

THREADS = 8
NEG_INF_F16 = 0xFC00


@pytest.fixture(scope="module")
def ll():
    b200.load()
    return importlib.import_module("llama_rust_b200.llama")


def make_model(ll, hp, seed, types=None):
    """{name: (type, blocks or f32 array, ne0, ne1)} with weights ~ N(0, 0.05) and norm weights near 1"""
    rng = np.random.default_rng(seed)
    tensors = {}
    for name, (ne0, ne1) in ll.tensor_shapes(hp).items():
        ty = types(name) if types else ll.q4_k_m_type(name, hp["n_layer"])
        if ty == orc.F32:
            arr = (1.0 + 0.1 * rng.standard_normal(ne0)).astype(np.float32)
        else:
            w = (rng.standard_normal((ne1, ne0)) * 0.05).astype(np.float32)
            arr = orc.quantize_rows(ty, w)
        tensors[name] = (ty, arr, ne0, ne1)
    return tensors


def both(ll, hp, tensors, n_ctx, n_batch):
    gpu = ll.Llama(hp, n_ctx, n_batch, cpu_threads=THREADS)
    for name, (ty, arr, ne0, ne1) in tensors.items():
        gpu.set_tensor(name, ty, arr, ne0, ne1)
    ohp = dict(n_vocab=hp["n_vocab"], n_embd=hp["n_embd"], n_head=hp["n_head"], n_head_kv=hp["n_head_kv"],
               head_dim=hp["n_embd_head"], n_ff=hp["n_ff"], n_layer=hp["n_layer"], rope_mode=hp["rope_mode"],
               n_ctx_orig=hp["n_ctx_train"], norm_eps=hp["norm_rms_eps"], freq_base=hp["rope_freq_base"],
               freq_scale=hp["rope_freq_scale"])
    cpu = orc_glue.Llama(ohp, {k: (v[0], v[1]) for k, v in tensors.items()}, n_ctx)
    return gpu, cpu


class CpuSession:
    """The cache bookkeeping of one sequence for the oracle: cells fill in order, n_kv pads to 256."""

    def __init__(self, cpu, n_ctx, wide):
        self.cpu, self.n_ctx, self.used, self.cell_pos, self.wide = cpu, n_ctx, 0, [], wide

    def decode(self, tokens, pos):
        n = len(tokens)
        head = self.used
        self.cell_pos += list(pos)
        self.used += n
        n_kv = min(self.n_ctx, max(256, (self.used + 255) // 256 * 256))
        mask = np.full((n, n_kv), NEG_INF_F16, dtype=np.uint16)
        cp = np.array(self.cell_pos)
        for i in range(n):
            mask[i, :self.used][cp <= pos[i]] = 0
        return self.cpu.forward(tokens, pos, n_kv, mask, np.arange(head, head + n), [n - 1], n_threads=THREADS,
                                wide_silu=self.wide)[0]


SMALL = dict(n_vocab=512, n_embd=512, n_head=8, n_head_kv=2, n_embd_head=64, n_ff=1024, n_layer=3, n_ctx_train=4096,
             rope_mode=0, norm_rms_eps=1e-5, rope_freq_base=10000.0, rope_freq_scale=1.0)
GQA128 = dict(n_vocab=1024, n_embd=1024, n_head=8, n_head_kv=2, n_embd_head=128, n_ff=2048, n_layer=2, n_ctx_train=8192,
              rope_mode=0, norm_rms_eps=1e-5, rope_freq_base=500000.0, rope_freq_scale=1.0)


def run_sequence(ll, hp, seed, prompt_len, n_gen, n_ctx=512, types=None):
    m = b200.load()
    wide = bool(m.lib.b200_host_silu_is_wide())
    tensors = make_model(ll, hp, seed, types)
    gpu, cpu = both(ll, hp, tensors, n_ctx, max(prompt_len, 1))
    sess = CpuSession(cpu, n_ctx, wide)
    rng = np.random.default_rng(seed + 1)
    prompt = rng.integers(0, hp["n_vocab"], prompt_len).astype(np.int32)
    pos = np.arange(prompt_len, dtype=np.int32)
    got, am = gpu.decode(prompt, pos, logits=True, argmax=True)
    want = sess.decode(prompt, pos)
    assert bits_equal(got, want), f"prompt logits differ: max |d| = {np.abs(got - want).max()}"
    assert am == orc_glue.argmax(want)
    tok = am
    for step in range(n_gen):
        p = prompt_len + step
        got, am = gpu.decode([tok], [p], logits=True, argmax=True)
        want = sess.decode(np.array([tok], dtype=np.int32), np.array([p], dtype=np.int32))
        assert bits_equal(got, want), f"step {step}: max |d| = {np.abs(got - want).max()}"
        assert am == orc_glue.argmax(want)
        tok = am
    assert gpu.kv_used() == prompt_len + n_gen
    gpu.close()


@pytest.mark.parametrize("prompt_len", [1, 5, 16, 70])
def test_small_model_prompt_then_greedy(ll, prompt_len):
    run_sequence(ll, SMALL, seed=10 + prompt_len, prompt_len=prompt_len, n_gen=6)


def test_gqa_head128_model(ll):
    run_sequence(ll, GQA128, seed=3, prompt_len=9, n_gen=4)


def test_crossing_a_256_cell_boundary(ll):
    # n_kv grows from 256 to 512 during generation: new graph, wider mask, split-KV chunks move
    run_sequence(ll, SMALL, seed=4, prompt_len=250, n_gen=10)


def test_q8_0_and_q4_0_model(ll):
    def types(name):
        if name.endswith("_norm.weight"):
            return orc.F32
        return orc.Q8_0 if (".attn_" in name or name == "output.weight") else orc.Q4_0
    run_sequence(ll, SMALL, seed=5, prompt_len=3, n_gen=3, types=types)


def test_kv_clear_restarts_the_sequence(ll):
    tensors = make_model(ll, SMALL, 6)
    gpu, _ = both(ll, SMALL, tensors, 256, 8)
    a = gpu.decode([1, 2, 3], [0, 1, 2])
    gpu.decode([4], [3])
    gpu.kv_clear()
    assert gpu.kv_used() == 0
    assert bits_equal(gpu.decode([1, 2, 3], [0, 1, 2]), a)
    gpu.close()


def test_argument_errors_are_statuses(ll):
    m = b200.load()
    tensors = make_model(ll, SMALL, 7)
    gpu, _ = both(ll, SMALL, tensors, 256, 4)
    with pytest.raises(m.B200Error, match="batch size"):
        gpu.decode([1, 2, 3, 4, 5], [0, 1, 2, 3, 4])
    with pytest.raises(m.B200Error, match="token"):
        gpu.decode([SMALL["n_vocab"]], [0])
    with pytest.raises(m.B200Error, match="bytes given"):
        gpu.set_tensor("output_norm.weight", orc.F32, np.zeros(3, dtype=np.float32), SMALL["n_embd"], 1)
    gpu.close()
    bad = dict(SMALL, n_embd_head=80)
    with pytest.raises(m.B200Error, match="head size"):
        ll.Llama(bad, 256, 4)


def test_launch_fusions_change_nothing(ll, monkeypatch):
    """sibling mat-muls in one launch, ROPE / SET_ROWS in one launch and the norm / silu / quantization in front of a
    one-row mat-mul inside its kernel (the defaults) against one launch per node: the same logits, prompt batch and
    single-token steps, with and without CUDA graphs"""
    tensors = make_model(ll, GQA128, 31)

    def run():
        gpu, _ = both(ll, GQA128, tensors, 512, 8)
        outs = [gpu.decode([5, 6, 7, 8, 9], [0, 1, 2, 3, 4])]
        for step in range(5):      # the third sight of a node list replays a captured graph
            outs.append(gpu.decode([10 + step], [5 + step]))
        gpu.close()
        return outs

    fused = run()
    monkeypatch.setenv("B200_FUSE_SIBLINGS", "0")
    monkeypatch.setenv("B200_FUSE_GLUE", "0")
    monkeypatch.setenv("B200_FUSE_PROLOGUE", "0")
    plain = run()
    monkeypatch.setenv("B200_CUDA_GRAPHS", "0")
    eager = run()
    for a, b, c in zip(fused, plain, eager):
        assert bits_equal(a, b) and bits_equal(a, c)


def test_gguf_file_loads_into_the_driver(ll, tmp_path):
    """a model written as a GGUF file and loaded by b200_llama_load_gguf answers like the same tensors set by hand"""
    gg = importlib.import_module("llama_rust_b200.gguf")
    tensors = make_model(ll, SMALL, 21)
    path = tmp_path / "small.gguf"
    gg.write_llama(path, SMALL, [(n, ty, arr, ne0, ne1) for n, (ty, arr, ne0, ne1) in tensors.items()])
    by_hand, _ = both(ll, SMALL, tensors, 256, 8)
    from_file = gg.load_llama(path, 256, 8, cpu_threads=THREADS)
    assert from_file.hp["n_layer"] == SMALL["n_layer"] and from_file.hp["n_vocab"] == SMALL["n_vocab"]
    assert from_file.hp["n_head_kv"] == SMALL["n_head_kv"] and from_file.hp["n_embd_head"] == SMALL["n_embd_head"]
    toks, pos = [3, 1, 4, 1, 5], [0, 1, 2, 3, 4]
    assert bits_equal(from_file.decode(toks, pos), by_hand.decode(toks, pos))
    assert bits_equal(from_file.decode([9], [5]), by_hand.decode([9], [5]))
    by_hand.close()
    from_file.close()
