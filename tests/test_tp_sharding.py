"""Tensor-parallel sharding (include/llama_b200.h, b200_tp_shard_*), on the CPU: the shards of every rank
put back together give the tensor back; row shards reproduce their rows of the mat-mul exactly; K shards'
partial sums add up to the whole within the stated 1e-5; and the same over two gloo ranks."""
import importlib
import os
import subprocess
import sys

import numpy as np
import pytest

import b200
import orc

HP = dict(n_vocab=512, n_embd=512, n_head=8, n_head_kv=2, n_embd_head=64, n_ff=1024, n_layer=1, n_ctx_train=4096, rope_mode=0,
          norm_rms_eps=1e-5, rope_freq_base=10000.0, rope_freq_scale=1.0)


@pytest.fixture(scope="module")
def ll():
    b200.load()
    return importlib.import_module("llama_rust_b200.llama")


def row_bytes(ty, ne0):
    return ne0 * 4 if ty == orc.F32 else orc.row_size(ty, ne0)


def model(ll, seed=0):
    rng = np.random.default_rng(seed)
    out = {}
    for name, (ne0, ne1) in ll.tensor_shapes(HP).items():
        ty = ll.q4_k_m_type(name, HP["n_layer"])
        if ty == orc.F32:
            out[name] = (ty, (1 + 0.1 * rng.standard_normal(ne0)).astype(np.float32).view(np.uint8), ne0, ne1)
        else:
            out[name] = (ty, orc.quantize_rows(ty, (rng.standard_normal((ne1, ne0)) * 0.05).astype(np.float32)).reshape(-1), ne0, ne1)
    return out


@pytest.mark.parametrize("tp", [2])
def test_shards_tile_the_tensor(ll, tp):
    for name, (ty, data, ne0, ne1) in model(ll).items():
        split, l0, l1 = ll.tp_shard_shape(name, ty, ne0, ne1, tp)
        shards = [ll.tp_shard_tensor(name, ty, data, ne0, ne1, r, tp) for r in range(tp)]
        whole = np.asarray(data, dtype=np.uint8).reshape(ne1, row_bytes(ty, ne0))
        if split == 0:
            assert (l0, l1) == (ne0, ne1) and all(np.array_equal(s, whole.ravel()) for s in shards), name
        elif split == 1:
            assert (l0, l1) == (ne0, ne1 // tp), name
            assert np.array_equal(np.concatenate([s.reshape(l1, -1) for s in shards]), whole), name
        else:
            assert (l0, l1) == (ne0 // tp, ne1), name
            assert np.array_equal(np.concatenate([s.reshape(ne1, -1) for s in shards], axis=1), whole), name
    kinds = {n.split(".")[-2]: ll.tp_shard_shape(n, t, a, b, tp)[0] for n, (t, _, a, b) in model(ll).items()}
    assert kinds["attn_q"] == kinds["attn_k"] == kinds["attn_v"] == kinds["ffn_gate"] == kinds["ffn_up"] == kinds["output"] == 1
    assert kinds["attn_output"] == kinds["ffn_down"] == 2 and kinds["token_embd"] == kinds["attn_norm"] == 0


def test_shapes_that_do_not_split_are_refused(ll):
    m = b200.load()
    with pytest.raises(m.B200Error, match="32-row"):
        ll.tp_shard_shape("blk.0.attn_k.weight", orc.Q4_K, 512, 80, 2)     # 40 rows per rank
    with pytest.raises(m.B200Error, match="256-element"):
        ll.tp_shard_shape("blk.0.ffn_down.weight", orc.Q4_K, 768, 512, 2)  # 384 columns per rank
    with pytest.raises(m.B200Error, match="heads"):
        ll.Llama(dict(HP, n_head_kv=1), 256, 4, tp_rank=0, tp_size=2, tp_id=bytes(128))


def partial_products(ll, name, ty, data, ne0, ne1, x, tp):
    """per rank: the oracle's mat-mul of the rank's shard with the activations it would see"""
    outs = []
    for r in range(tp):
        split, l0, l1 = ll.tp_shard_shape(name, ty, ne0, ne1, tp)
        w = ll.tp_shard_tensor(name, ty, data, ne0, ne1, r, tp).reshape(l1, -1)
        xr = x if split != 2 else np.ascontiguousarray(x[:, r * l0:(r + 1) * l0])
        outs.append(orc.mul_mat(ty, w, xr)[0])
    return outs


@pytest.mark.parametrize("m_rows", [1, 5])
def test_row_shards_are_exact_and_k_shards_sum_within_tolerance(ll, m_rows):
    tensors = model(ll, seed=1)
    rng = np.random.default_rng(2)
    for name in ("blk.0.attn_q.weight", "blk.0.ffn_up.weight", "blk.0.attn_output.weight", "blk.0.ffn_down.weight"):
        ty, data, ne0, ne1 = tensors[name]
        x = rng.standard_normal((m_rows, ne0)).astype(np.float32)
        whole = orc.mul_mat(ty, np.asarray(data).reshape(ne1, -1), x)[0]
        parts = partial_products(ll, name, ty, data, ne0, ne1, x, 2)
        if ll.tp_shard_shape(name, ty, ne0, ne1, 2)[0] == 1:
            assert np.array_equal(np.concatenate(parts, axis=1).view(np.uint32), whole.view(np.uint32)), name
        else:
            got = parts[0] + parts[1]
            assert np.abs(got - whole).max() <= 1e-5 * np.abs(whole).max(), name


RANK_SCRIPT = r"""
import os, sys, importlib
import numpy as np
sys.path.insert(0, os.path.join(os.environ["REPO"], "tests"))
import torch, torch.distributed as dist
import b200, orc
import test_tp_sharding as T
b200.load()
ll = importlib.import_module("llama_rust_b200.llama")
dist.init_process_group(backend="gloo")
rank, world = dist.get_rank(), dist.get_world_size()
tensors = T.model(ll, seed=1)
rng = np.random.default_rng(2)
ok = True
for name in ("blk.0.attn_output.weight", "blk.0.ffn_down.weight"):
    ty, data, ne0, ne1 = tensors[name]
    x = rng.standard_normal((1, ne0)).astype(np.float32)
    split, l0, l1 = ll.tp_shard_shape(name, ty, ne0, ne1, world)
    w = ll.tp_shard_tensor(name, ty, data, ne0, ne1, rank, world).reshape(l1, -1)
    part = torch.from_numpy(orc.mul_mat(ty, w, np.ascontiguousarray(x[:, rank * l0:(rank + 1) * l0]))[0].copy())
    dist.all_reduce(part)     # what the NCCL all-reduce does after attn_output / ffn_down
    whole = orc.mul_mat(ty, np.asarray(data).reshape(ne1, -1), x)[0]
    ok = ok and float(np.abs(part.numpy() - whole).max()) <= 1e-5 * float(np.abs(whole).max())
flag = torch.tensor([1 if ok else 0])
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 1)
"""


def test_k_split_over_two_gloo_ranks(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT)
    env = dict(os.environ, REPO=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29631", str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
