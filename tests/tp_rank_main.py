"""One rank of the tensor-parallel GPU test (launched by tests/test_gpu_tp.py through torch.distributed.run):
a small Llama split over the ranks' GPUs against the same model on one GPU."""
import importlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import torch
import torch.distributed as dist

import b200
import test_gpu_llama as T


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

    hp = dict(T.GQA128, n_head_kv=2 if world <= 2 else world, n_head=8 if world <= 8 else world)
    tensors = T.make_model(ll, hp, seed=42)
    tp = ll.Llama(hp, 512, max(16, int(os.environ.get("TP_PROMPT", "9"))), device=rank, cpu_threads=T.THREADS, tp_rank=rank, tp_size=world, tp_id=ident)
    for name, (ty, arr, ne0, ne1) in tensors.items():
        tp.set_tensor(name, ty, arr, ne0, ne1)
    one = None
    if rank == 0:
        one = ll.Llama(hp, 512, max(16, int(os.environ.get("TP_PROMPT", "9"))), device=0, cpu_threads=T.THREADS)
        for name, (ty, arr, ne0, ne1) in tensors.items():
            one.set_tensor(name, ty, arr, ne0, ne1)
    rng = np.random.default_rng(7)
    n_prompt = int(os.environ.get("TP_PROMPT", "9"))
    prompt = rng.integers(0, hp["n_vocab"], n_prompt).astype(np.int32)
    ok, worst, diverged = True, 0.0, None
    toks, pos = prompt, np.arange(n_prompt, dtype=np.int32)
    for step in range(8):
        if os.environ.get("TP_BARRIER"):
            dist.barrier()
        got, am = tp.decode(toks, pos, logits=True, argmax=True)
        nxt = np.array([am], dtype=np.int32)
        if rank == 0:
            want, am1 = one.decode(toks, pos, logits=True, argmax=True)
            err = float(np.abs(got - want).max() / np.abs(want).max())
            worst = max(worst, err)
            # A K-split changes the order of the f32 partial sums (1e-7), and the next Q8_K quantization turns a
            # few of those last-bit differences into one-step differences of a quant: the logits agree to the
            # activation-quantization noise, not to the mat-mul tolerance.  Greedy tokens are compared and the
            # first divergence is reported.
            ok = ok and err <= 5e-2
            if am != am1 and diverged is None:
                diverged = step
        toks, pos = nxt, np.array([n_prompt + step], dtype=np.int32)
    # every rank must hold the same gathered logits / token
    t = torch.tensor([float(am)], device="cuda")
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ok = ok and float(lo.item()) == float(hi.item())
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"tp{world}: worst relative logit error {worst:.3e}, first greedy divergence at step {diverged}, ok={bool(flag.item())}", flush=True)
    tp.close()
    if one is not None:
        one.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
