"""Structure check of the oracle's Llama forward: a float64 numpy decoder over the dequantized weights
(no activation quantization, plain softmax attention) must land close to it.  The op-level arithmetic
is pinned elsewhere (golden vectors); this guards the wiring: rope pairing, GQA head mapping, cache
rows, mask, residuals."""
import numpy as np

import orc
import orc_glue

HP = dict(n_vocab=256, n_embd=256, n_head=4, n_head_kv=2, head_dim=64, n_ff=512, n_layer=2, rope_mode=0, n_ctx_orig=4096,
          norm_eps=1e-5, freq_base=10000.0, freq_scale=1.0)


def shapes(hp):
    E, FF, V = hp["n_embd"], hp["n_ff"], hp["n_vocab"]
    EQ, EK = hp["n_head"] * hp["head_dim"], hp["n_head_kv"] * hp["head_dim"]
    s = {"token_embd.weight": (E, V), "output_norm.weight": (E, 1), "output.weight": (E, V)}
    for il in range(hp["n_layer"]):
        p = f"blk.{il}."
        s.update({p + "attn_norm.weight": (E, 1), p + "attn_q.weight": (E, EQ), p + "attn_k.weight": (E, EK),
                  p + "attn_v.weight": (E, EK), p + "attn_output.weight": (EQ, E), p + "ffn_norm.weight": (E, 1),
                  p + "ffn_gate.weight": (E, FF), p + "ffn_up.weight": (E, FF), p + "ffn_down.weight": (FF, E)})
    return s


def make(hp, seed):
    rng = np.random.default_rng(seed)
    q, dense = {}, {}
    for name, (ne0, ne1) in shapes(hp).items():
        if name.endswith("_norm.weight"):
            w = (1.0 + 0.1 * rng.standard_normal(ne0)).astype(np.float32)
            q[name], dense[name] = (orc.F32, w), w.astype(np.float64)
        else:
            ty = orc.Q6_K if ("attn_v" in name or name == "output.weight") else orc.Q4_K
            w = (rng.standard_normal((ne1, ne0)) * 0.05).astype(np.float32)
            blocks = orc.quantize_rows(ty, w)
            q[name], dense[name] = (ty, blocks), orc.dequantize(ty, blocks, ne0).astype(np.float64)
    return q, dense


def rope64(x, pos, base):
    # x: [T, H, D], adjacent pairs (mode 0)
    D = x.shape[-1]
    inv = base ** (-np.arange(0, D, 2) / D)
    ang = pos[:, None, None] * inv[None, None, :]
    c, s = np.cos(ang), np.sin(ang)
    y = np.empty_like(x)
    y[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
    y[..., 1::2] = x[..., 0::2] * s + x[..., 1::2] * c
    return y


def forward64(hp, w, tokens):
    T = len(tokens)
    H, HK, D = hp["n_head"], hp["n_head_kv"], hp["head_dim"]
    pos = np.arange(T, dtype=np.float64)

    def norm(x, g):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + hp["norm_eps"]) * g

    x = w["token_embd.weight"][tokens]
    for il in range(hp["n_layer"]):
        p = f"blk.{il}."
        h = norm(x, w[p + "attn_norm.weight"])
        q = rope64((h @ w[p + "attn_q.weight"].T).reshape(T, H, D), pos, hp["freq_base"])
        k = rope64((h @ w[p + "attn_k.weight"].T).reshape(T, HK, D), pos, hp["freq_base"])
        v = (h @ w[p + "attn_v.weight"].T).reshape(T, HK, D)
        att = np.empty((T, H, D))
        for hd in range(H):
            kv = hd // (H // HK)
            s = q[:, hd] @ k[:, kv].T / np.sqrt(D)
            s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
            pr = np.exp(s - s.max(-1, keepdims=True))
            att[:, hd] = (pr / pr.sum(-1, keepdims=True)) @ v[:, kv]
        x = x + att.reshape(T, H * D) @ w[p + "attn_output.weight"].T
        h = norm(x, w[p + "ffn_norm.weight"])
        g = h @ w[p + "ffn_gate.weight"].T
        x = x + ((g / (1 + np.exp(-g))) * (h @ w[p + "ffn_up.weight"].T)) @ w[p + "ffn_down.weight"].T
    return norm(x, w["output_norm.weight"]) @ w["output.weight"].T


def oracle_logits(model, tokens, n_ctx=256, split=None):
    """all tokens in one batch, or (split) a prompt batch followed by single-token steps"""
    T = len(tokens)
    out = []
    steps = [(0, T)] if split is None else [(0, split)] + [(i, i + 1) for i in range(split, T)]
    for a, b in steps:
        n = b - a
        mask = np.full((n, 256), 0xFC00, dtype=np.uint16)
        for i in range(n):
            mask[i, :a + i + 1] = 0
        out.append(model.forward(tokens[a:b], np.arange(a, b), 256, mask, np.arange(a, b), np.arange(n), n_threads=4))
    return np.concatenate(out)


def test_oracle_llama_tracks_a_float64_decoder():
    q, dense = make(HP, 0)
    tokens = np.random.default_rng(1).integers(0, HP["n_vocab"], 12).astype(np.int32)
    want = forward64(HP, dense, tokens)
    got = oracle_logits(orc_glue.Llama(HP, q, 256), tokens)
    err = np.abs(got - want).max() / np.abs(want).max()
    assert err < 5e-2, err   # Q8 activations and the F16 cache cost about 2 %; a wiring error costs 100 %
    assert (got.argmax(-1) == want.argmax(-1)).mean() >= 0.9


def test_prompt_plus_steps_tracks_one_batch():
    # different mat-mul / attention routes for the same tokens: same function, slightly different rounding
    q, _ = make(HP, 2)
    tokens = np.random.default_rng(3).integers(0, HP["n_vocab"], 10).astype(np.int32)
    whole = oracle_logits(orc_glue.Llama(HP, q, 256), tokens)
    stepped = oracle_logits(orc_glue.Llama(HP, q, 256), tokens, split=6)
    assert np.abs(whole - stepped).max() / np.abs(whole).max() < 2e-2


def test_tensor_parallel_forward_restatement():
    """orc_llama_forward_tp: with one rank it is the plain forward bit for bit; with two or four ranks the K-split
    partial results of layer 0 add up, in rank order, to what the layer then uses, and the logits stay within the
    activation-quantization noise of the unsplit model (a last-bit change of a partial sum can flip a Q8 rounding
    in the next layer)."""
    hp = dict(HP, n_embd=1024, n_head=16, n_head_kv=4, n_ff=1024)   # a quarter of the heads / FFN rows is 256 columns
    q, _ = make(hp, 4)
    tokens = np.random.default_rng(5).integers(0, hp["n_vocab"], 7).astype(np.int32)
    n = len(tokens)
    mask = np.full((n, 256), 0xFC00, dtype=np.uint16)
    for i in range(n):
        mask[i, :i + 1] = 0
    args = (tokens, np.arange(n), 256, mask, np.arange(n), np.arange(n))
    plain = orc_glue.Llama(hp, q, 256).forward(*args, n_threads=4)
    one = orc_glue.Llama(hp, q, 256).forward_tp(*args, tp=1, n_threads=4)
    assert np.array_equal(plain.view(np.uint32), one.view(np.uint32))
    for tp in (2, 4):
        logits, pa, pf = orc_glue.Llama(hp, q, 256).forward_tp(*args, tp=tp, n_threads=4, partials=True)
        assert np.abs(logits - plain).max() / np.abs(plain).max() < 5e-2
        assert pa.shape == (tp, n, hp["n_embd"]) and np.abs(pa).max() > 0 and np.abs(pf).max() > 0
