"""MUL_MAT_ID on the GPU vs the CPU oracle and the reference's dump, through the C ABI (-m gpu)."""
import numpy as np
import pytest

import b200
import orc
import synth
from conftest import bits_equal

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


def top_k_ids(n_tok, n_expert, k, seed):
    """k expert ids per token, uniform without replacement (a partial Fisher-Yates per token)."""
    rng = np.random.default_rng(seed)
    return np.stack([rng.permutation(n_expert)[:k] for _ in range(n_tok)]).astype(np.int32)


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K"])
def test_reference_dump_tiled_and_row_dot_experts(dev, golden, name):
    """5 experts of 140 rows (not a multiple of 8): four take the tiled chain, the one with 6 routed
    rows the row dot (crates/ggml/src/compute.rs:2036-2104,2183-2190)."""
    g = golden("tiled")
    ty = {"Q4_K": orc.Q4_K, "Q6_K": orc.Q6_K}[name]
    W, B, ids, dst = (g[f"mmid/{name}/{x}"] for x in ("W", "B", "ids", "dst"))
    n_as, n, _ = W.shape
    w = dev.ExpertWeights(ty, W, n, B.shape[2])
    assert bits_equal(dev.mul_mat_id(w, B, ids), dst)


@pytest.mark.parametrize("ne11", [1, 8])
def test_mxfp4_experts_full_size(dev, ne11):
    """128 experts of 768 x 2048 MXFP4, 512 tokens, top-8: the gate/up form (one activation row per
    token) and the down form (one row per slot, i11 = slot)."""
    E, n, k, n_tok, top = 128, 768, 2048, 512, 8
    W = synth.weights(orc.MXFP4, E * n, k, seed=61, period=8 * n).reshape(E, n, -1)
    B = synth.activations(n_tok * ne11, k, seed=62).reshape(n_tok, ne11, k)
    ids = top_k_ids(n_tok, E, top, seed=63)
    want, route = orc.mul_mat_id(orc.MXFP4, W, B, ids)
    assert route == orc.ROUTE_REPACK
    got = dev.mul_mat_id(dev.ExpertWeights(orc.MXFP4, W, n, k), B, ids)
    assert bits_equal(got, want)


@pytest.mark.parametrize("ty", [orc.Q4_K, orc.Q4_0, orc.Q8_0], ids=lambda t: orc.TYPE_NAMES[t])
def test_other_expert_types(dev, ty):
    E, n, k, n_tok, top = 6, 64, 512, 9, 2
    W = synth.weights(ty, E * n, k, seed=71).reshape(E, n, -1)
    B = synth.activations(n_tok * top, k, seed=72).reshape(n_tok, top, k)
    ids = top_k_ids(n_tok, E, top, seed=73)
    want, _ = orc.mul_mat_id(ty, W, B, ids)
    got = dev.mul_mat_id(dev.ExpertWeights(ty, W, n, k), B, ids)
    assert bits_equal(got, want)


def test_empty_batch(dev):
    W = synth.weights(orc.MXFP4, 2 * 32, 256, seed=1).reshape(2, 32, -1)
    w = dev.ExpertWeights(orc.MXFP4, W, 32, 256)
    out = dev.mul_mat_id(w, np.zeros((0, 1, 256), np.float32), np.zeros((0, 2), np.int32))
    assert out.shape == (0, 2, 32)


@pytest.mark.parametrize("ty", [orc.MXFP4, orc.Q4_0], ids=lambda t: orc.TYPE_NAMES[t])
def test_grouped_by_expert_with_ragged_counts(dev, ty):
    """enough pairs for the expert-grouped tensor-core path: one expert gets far more than 32 pairs (several work
    items, the last one short), one gets none, the pair count is not a multiple of 32"""
    E, n, k, n_tok, top = 7, 96, 512, 71, 3
    W = synth.weights(ty, E * n, k, seed=81).reshape(E, n, -1)
    B = synth.activations(n_tok * top, k, seed=82).reshape(n_tok, top, k)
    rng = np.random.default_rng(83)
    ids = np.empty((n_tok, top), dtype=np.int32)
    for t in range(n_tok):
        # expert 0 in most tokens, expert 5 never; ids of a token are distinct
        pool = [e for e in range(E) if e != 5]
        chosen = [0] if t % 5 else []
        rest = [e for e in pool if e not in chosen]
        chosen += list(rng.permutation(rest)[:top - len(chosen)])
        ids[t] = chosen
    want, route = orc.mul_mat_id(ty, W, B, ids)
    assert route == orc.ROUTE_REPACK
    got = dev.mul_mat_id(dev.ExpertWeights(ty, W, n, k), B, ids)
    assert dev.kernel_error() == 0
    assert bits_equal(got, want)
