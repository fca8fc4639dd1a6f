"""Several sequences in one decode step (b200_llama_decode_seqs): prompts of different lengths go in one by
one, then every step carries one token per sequence.  Logits of every sequence are compared bit for bit with
the CPU oracle's forward over the same unified cache (same cells, same mask)."""
import importlib

import numpy as np
import pytest

import b200
import orc_glue
import test_gpu_llama as T
from conftest import bits_equal

pytestmark = pytest.mark.gpu


class CpuCache:
    """the unified cache bookkeeping for the oracle: next free cells, (sequence, position) per cell"""

    def __init__(self, cpu, n_ctx, wide):
        self.cpu, self.n_ctx, self.wide = cpu, n_ctx, wide
        self.seq, self.pos = [], []

    def decode(self, tokens, pos, seqs, out_rows):
        n, head = len(tokens), len(self.seq)
        self.seq += list(seqs)
        self.pos += list(pos)
        used = len(self.seq)
        n_kv = min(self.n_ctx, max(256, (used + 255) // 256 * 256))
        mask = np.full((n, n_kv), T.NEG_INF_F16, dtype=np.uint16)
        cs, cp = np.array(self.seq), np.array(self.pos)
        for i in range(n):
            mask[i, :used][(cs == seqs[i]) & (cp <= pos[i])] = 0
        return self.cpu.forward(tokens, pos, n_kv, mask, np.arange(head, head + n), out_rows, n_threads=T.THREADS, wide_silu=self.wide)


@pytest.mark.parametrize("n_seq,steps", [(3, 5), (16, 3)])
def test_parallel_sequences_match_the_cpu(n_seq, steps):
    m = b200.load()
    ll = importlib.import_module("llama_rust_b200.llama")
    wide = bool(m.lib.b200_host_silu_is_wide())
    hp = T.SMALL
    tensors = T.make_model(ll, hp, seed=100 + n_seq)
    gpu, cpu = T.both(ll, hp, tensors, 1024, 32)
    cache = CpuCache(cpu, 1024, wide)
    rng = np.random.default_rng(n_seq)
    lens = rng.integers(2, 12, n_seq)
    nxt = np.zeros(n_seq, dtype=np.int32)
    for s in range(n_seq):   # prompts, one sequence per call
        toks = rng.integers(0, hp["n_vocab"], lens[s]).astype(np.int32)
        pos = np.arange(lens[s], dtype=np.int32)
        got, am = gpu.decode_seqs(toks, pos, np.full(lens[s], s), [lens[s] - 1], logits=True, argmax=True)
        want = cache.decode(toks, pos, [s] * int(lens[s]), [lens[s] - 1])
        assert bits_equal(got, want), f"prompt of sequence {s}"
        nxt[s] = am[0]
    for step in range(steps):   # one token per sequence per step
        pos = (lens + step).astype(np.int32)
        got, am = gpu.decode_seqs(nxt, pos, np.arange(n_seq), np.arange(n_seq), logits=True, argmax=True)
        want = cache.decode(nxt, pos, list(range(n_seq)), np.arange(n_seq))
        assert bits_equal(got, want), f"step {step}: max |d| = {np.abs(got - want).max()}"
        assert list(am) == [orc_glue.argmax(r) for r in want]
        nxt = am.astype(np.int32)
    assert gpu.kv_used() == int(lens.sum()) + n_seq * steps
    gpu.close()


def test_sequences_do_not_see_each_other():
    """a sequence decoded next to others gets the logits it gets alone (its mask hides the other cells);
    bit-exact only where the routes agree, so both runs use the same batch shapes"""
    ll = importlib.import_module("llama_rust_b200.llama")
    hp = T.SMALL
    tensors = T.make_model(ll, hp, seed=77)
    rng = np.random.default_rng(5)
    a = rng.integers(0, hp["n_vocab"], 6).astype(np.int32)
    b = rng.integers(0, hp["n_vocab"], 6).astype(np.int32)
    outs = []
    for other in (b, a[::-1].copy()):   # sequence 0 next to two different neighbours
        gpu, _ = T.both(ll, hp, tensors, 512, 16)
        toks = np.concatenate([a, other])
        pos = np.concatenate([np.arange(6), np.arange(6)])
        seqs = np.array([0] * 6 + [1] * 6)
        logits, _ = gpu.decode_seqs(toks, pos, seqs, [5], logits=True)
        outs.append(logits[0])
        gpu.close()
    assert bits_equal(outs[0], outs[1])
