"""A two-layer model of the Llama-3-8B shape (d_model 4096, 32 query heads on 8 KV heads of 128, FFN 14336,
Q4_K_M tensor types; the vocabulary cut to 4096 rows to keep the CPU side short) through the decode driver:
a 256-token prompt batch, where the library's time model sends the Q4_K mat-muls to the two-pass tcgen05
kernels, then greedy single-token steps.  Logits bit for bit against the CPU oracle's forward; the greedy token
streams must be identical."""
import importlib

import numpy as np
import pytest

import b200
import orc_glue
import test_gpu_llama as T
from conftest import bits_equal

pytestmark = pytest.mark.gpu


def test_two_layers_of_the_8b_shape_prompt_256_then_greedy():
    dev = b200.load()
    assert dev.device_count() > 0
    dev.set_device(0)
    ll = importlib.import_module("llama_rust_b200.llama")
    hp = dict(ll.LLAMA3_8B, n_layer=2, n_vocab=4096)
    # layer 0: attn_v / ffn_down Q6_K (use_more_bits), layer 1 likewise for a 2-layer model; output Q6_K
    tensors = T.make_model(ll, hp, seed=808)
    n_ctx, n_prompt, n_gen = 512, 256, 4
    # the prompt shape is one the time model gives to the two-pass kernels (host arithmetic, no CUDA call)
    assert dev.lib.b200_prompt_kernel_choice(4096, n_prompt, 148) in (3, 4)
    assert dev.lib.b200_prompt_kernel_choice(14336, n_prompt, 148) in (3, 4)
    gpu, cpu = T.both(ll, hp, tensors, n_ctx, n_prompt)
    sess = T.CpuSession(cpu, n_ctx, bool(dev.lib.b200_host_silu_is_wide()))
    prompt = np.random.default_rng(809).integers(0, hp["n_vocab"], n_prompt).astype(np.int32)
    pos = np.arange(n_prompt, dtype=np.int32)
    got, am = gpu.decode(prompt, pos, logits=True, argmax=True)
    want = sess.decode(prompt, pos)
    assert dev.kernel_error() == 0
    assert bits_equal(got, want), f"prompt logits: max |d| = {np.abs(got - want).max()}"
    gpu_stream, cpu_stream = [am], [orc_glue.argmax(want)]
    for i in range(n_gen):
        p = n_prompt + i
        got, am = gpu.decode([gpu_stream[-1]], [p], logits=True, argmax=True)
        want = sess.decode(np.array([cpu_stream[-1]], dtype=np.int32), np.array([p], dtype=np.int32))
        assert bits_equal(got, want), f"step {i}: max |d| = {np.abs(got - want).max()}"
        gpu_stream.append(am)
        cpu_stream.append(orc_glue.argmax(want))
    assert gpu_stream == cpu_stream
    gpu.close()
