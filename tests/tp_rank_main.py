"""One rank of the tensor-parallel GPU test (launched by tests/test_gpu_tp.py through torch.distributed.run):
a small Llama split over the ranks' GPUs against the CPU restatement of the same cut (orc_llama_forward_tp: the
partial results of attn_output / ffn_down added in rank order).  The library's peer-memory all-reduce adds in that
order for any number of ranks, and with two ranks any all-reduce does (a + b is order-free), so the logits of every
step must equal the restatement's bit for bit and the greedy tokens must be the same; only a group of more than two
ranks that fell back to NCCL is compared within a bound instead (NCCL's order is its own)."""
import importlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import torch
import torch.distributed as dist

import b200
import orc_glue
import test_gpu_llama as T
from test_gpu_tp_one_gpu import cpu_session


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group(backend="nccl")
    m = b200.load()
    m.set_device(rank)
    ll = importlib.import_module("llama_rust_b200.llama")
    # the group id: made on rank 0, broadcast as bytes
    ident = torch.zeros(128, dtype=torch.uint8, device="cuda")
    if rank == 0:
        ident = torch.tensor(list(ll.tp_unique_id()), dtype=torch.uint8, device="cuda")
    dist.broadcast(ident, 0)
    ident = bytes(ident.cpu().tolist())

    hp = dict(T.GQA128, n_head_kv=max(2, world), n_head=8 if world <= 8 else world)
    tensors = T.make_model(ll, hp, seed=42)
    n_prompt = int(os.environ.get("TP_PROMPT", "9"))
    tp = ll.Llama(hp, 512, max(16, n_prompt), device=rank, cpu_threads=T.THREADS, tp_rank=rank, tp_size=world, tp_id=ident)
    for name, (ty, arr, ne0, ne1) in tensors.items():
        tp.set_tensor(name, ty, arr, ne0, ne1)
    kind = tp.tp_exchange_kind()
    exact = kind == 1 or world == 2
    cpu_step = cpu_session(hp, tensors, 512, bool(m.lib.b200_host_silu_is_wide()), world) if rank == 0 else None
    rng = np.random.default_rng(7)
    prompt = rng.integers(0, hp["n_vocab"], n_prompt).astype(np.int32)
    ok, worst, diverged = True, 0.0, None
    toks, pos = prompt, np.arange(n_prompt, dtype=np.int32)
    for step in range(8):    # the third single-token step replays a captured CUDA graph
        got, am = tp.decode(toks, pos, logits=True, argmax=True)
        nxt = np.array([am], dtype=np.int32)
        if rank == 0:
            want, _, _ = cpu_step(toks, pos)
            err = float(np.abs(got - want).max() / np.abs(want).max())
            worst = max(worst, err)
            same = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
            ok = ok and (same if exact else err <= 1e-3)
            if am != orc_glue.argmax(want) and diverged is None:
                diverged = step
                ok = ok and not exact
        toks, pos = nxt, np.array([n_prompt + step], dtype=np.int32)
    ok = ok and m.kernel_error() == 0
    # every rank must hold the same gathered logits / token
    t = torch.tensor([float(am)], device="cuda")
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ok = ok and float(lo.item()) == float(hi.item())
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"tp{world}: exchange kind {kind} ({'peer-memory kernel' if kind == 1 else 'NCCL'}), worst relative logit error vs the CPU cut "
              f"{worst:.3e}, first greedy divergence at step {diverged}, ok={bool(flag.item())}", flush=True)
    tp.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
