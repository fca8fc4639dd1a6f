"""Row-split tensor parallelism checked bit for bit on ONE GPU.

Each rank of a tensor-parallel group is a decode driver of its own (its shard of every matrix, its heads' KV cache).
Here the ranks of a group run as threads of this process on the same GPU, and the collectives between them are
carried out on the host through the driver's exchange hook (b200_llama_new_tp_hook): the partial sums are added in
rank order, which is what the library's peer-memory all-reduce does between real GPUs.  What is checked, against
the CPU restatement of the same cut (orc_llama_forward_tp):

* rank r's partial result of layer 0's attn_output and ffn_down, before any exchange: the cut itself (which rows,
  which K columns, which heads, which activation blocks);
* the logits every rank ends up with, prompt batch and greedy single-token steps, and the greedy tokens.

All comparisons are exact (same bits).  Two and four ranks: with four, the order of the additions matters.
"""
import importlib
import threading

import numpy as np
import pytest

import b200
import orc
import orc_glue
import test_gpu_llama as T
from conftest import bits_equal

pytestmark = pytest.mark.gpu


class HostExchange:
    """the hook of every rank: a rendezvous of the rank threads around host copies of the operands"""

    def __init__(self, dev, size):
        self.dev, self.size = dev, size
        self.barrier = threading.Barrier(size, timeout=120)
        # The library is driven from one thread at a time (its scratch blocks are per device, not per driver): a rank
        # thread holds this lock while it issues GPU work and lends it to the others while it waits in the hook, which
        # the driver enters with its stream drained.
        self.turn = threading.Lock()
        self.parts = [None] * size
        self.reduces = []          # per all-reduce of the current step: the ranks' partial operands
        self.failed = None

    def _down(self, ptr, count):
        out = np.empty(count, dtype=np.float32)
        self.dev.check(self.dev.lib.b200_memcpy_d2h(out.ctypes.data, ptr, out.nbytes, None), "d2h")
        return out

    def _up(self, ptr, arr):
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        self.dev.check(self.dev.lib.b200_memcpy_h2d(ptr, arr.ctypes.data, arr.nbytes, None), "h2d")
        self.dev.synchronize()

    def __call__(self, kind, rank, size, buf, count, dst, n_local, rows):
        held = True                   # the calling rank thread holds the turn lock on entry and must on return

        def rendezvous():
            nonlocal held
            self.turn.release()
            held = False
            self.barrier.wait()
            self.turn.acquire()
            held = True

        try:
            self.parts[rank] = self._down(buf, count)
            rendezvous()
            if kind == 0:
                total = self.parts[0].copy()
                for r in range(1, size):
                    total = total + self.parts[r]        # f32 adds in rank order
                self._up(buf, total)
                if rank == 0:
                    self.reduces.append([p.copy() for p in self.parts])
            else:
                out = np.empty((rows, n_local * size), dtype=np.float32)
                for r in range(size):
                    out[:, r * n_local:(r + 1) * n_local] = self.parts[r].reshape(rows, n_local)
                self._up(dst, out)
            rendezvous()              # nobody overwrites parts[] before everybody has read them
            return 0
        except Exception as exc:      # a ctypes callback must not raise
            self.failed = exc
            self.barrier.abort()
            if not held:
                self.turn.acquire()
            return 1


def cpu_session(hp, tensors, n_ctx, wide, tp):
    ohp = dict(n_vocab=hp["n_vocab"], n_embd=hp["n_embd"], n_head=hp["n_head"], n_head_kv=hp["n_head_kv"],
               head_dim=hp["n_embd_head"], n_ff=hp["n_ff"], n_layer=hp["n_layer"], rope_mode=hp["rope_mode"],
               n_ctx_orig=hp["n_ctx_train"], norm_eps=hp["norm_rms_eps"], freq_base=hp["rope_freq_base"],
               freq_scale=hp["rope_freq_scale"])
    cpu = orc_glue.Llama(ohp, {k: (v[0], v[1]) for k, v in tensors.items()}, n_ctx)
    state = {"used": 0, "cell_pos": []}

    def step(tokens, pos):
        n = len(tokens)
        head = state["used"]
        state["cell_pos"] += list(pos)
        state["used"] += n
        n_kv = min(n_ctx, max(256, (state["used"] + 255) // 256 * 256))
        mask = np.full((n, n_kv), T.NEG_INF_F16, dtype=np.uint16)
        cp = np.array(state["cell_pos"])
        for i in range(n):
            mask[i, :state["used"]][cp <= pos[i]] = 0
        logits, pa, pf = cpu.forward_tp(tokens, pos, n_kv, mask, np.arange(head, head + n), [n - 1], tp, n_threads=T.THREADS,
                                        wide_silu=wide, partials=True)
        return logits[0], pa, pf

    return step


@pytest.mark.parametrize("tp", [2, 4])
def test_ranks_as_threads_match_the_cpu_cut_bit_for_bit(tp):
    dev = b200.load()
    assert dev.device_count() > 0
    dev.set_device(0)
    ll = importlib.import_module("llama_rust_b200.llama")
    hp = dict(T.GQA128, n_head_kv=max(2, tp), n_head=8)
    tensors = T.make_model(ll, hp, seed=90 + tp)
    n_ctx, n_prompt, n_gen = 512, 9, 4
    ex = HostExchange(dev, tp)
    ranks = []
    for r in range(tp):
        g = ll.Llama(hp, n_ctx, 16, device=0, cpu_threads=T.THREADS, tp_rank=r, tp_size=tp, tp_hook=ex)
        for name, (ty, arr, ne0, ne1) in tensors.items():
            g.set_tensor(name, ty, arr, ne0, ne1)       # the whole tensor: the driver keeps this rank's shard
        ranks.append(g)
    assert ranks[0].tp_exchange_kind() == -1
    cpu_step = cpu_session(hp, tensors, n_ctx, bool(dev.lib.b200_host_silu_is_wide()), tp)

    def step(tokens, pos):
        tokens, pos = np.asarray(tokens, dtype=np.int32), np.asarray(pos, dtype=np.int32)
        ex.reduces.clear()
        out = [None] * tp

        def run(r):
            try:
                with ex.turn:
                    dev.set_device(0)
                    out[r] = ranks[r].decode(tokens, pos, logits=True, argmax=True)
            except Exception as exc:
                out[r] = exc
                ex.barrier.abort()

        threads = [threading.Thread(target=run, args=(r,)) for r in range(tp)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert ex.failed is None, ex.failed
        for o in out:
            assert not isinstance(o, Exception), o
        want, pa, pf = cpu_step(tokens, pos)
        # layer 0: the first two all-reduces of the step saw these partial operands
        for r in range(tp):
            assert bits_equal(ex.reduces[0][r], pa[r].ravel()), f"attn_output partial of rank {r}"
            assert bits_equal(ex.reduces[1][r], pf[r].ravel()), f"ffn_down partial of rank {r}"
        assert len(ex.reduces) == 2 * hp["n_layer"]
        for r in range(tp):
            logits, am = out[r]
            assert bits_equal(logits, want), f"rank {r}: max |d| = {np.abs(logits - want).max()}"
            assert am == orc_glue.argmax(want)
        return out[0][1]

    rng = np.random.default_rng(7)
    tok = step(rng.integers(0, hp["n_vocab"], n_prompt), np.arange(n_prompt))
    for i in range(n_gen):
        tok = step([tok], [n_prompt + i])
    for g in ranks:
        g.close()
