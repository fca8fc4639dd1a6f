"""Shapes and tensor types of llama-architecture models.  Pure Python: this module is importable on its own
(by path), without the CUDA library, so that a CPU-only process can build the same synthetic models."""

F32, Q4_K, Q6_K = 0, 12, 14

# Llama-3-70B shape (BASELINE's tensor-parallel configuration)
LLAMA3_70B = dict(n_vocab=128256, n_embd=8192, n_head=64, n_head_kv=8, n_embd_head=128, n_ff=28672, n_layer=80,
                  n_ctx_train=8192, rope_mode=0, norm_rms_eps=1e-5, rope_freq_base=500000.0, rope_freq_scale=1.0)

# Llama-3-8B (BASELINE configuration of the tokens/s metric)
LLAMA3_8B = dict(n_vocab=128256, n_embd=4096, n_head=32, n_head_kv=8, n_embd_head=128, n_ff=14336, n_layer=32,
                 n_ctx_train=8192, rope_mode=0, norm_rms_eps=1e-5, rope_freq_base=500000.0, rope_freq_scale=1.0)


def use_more_bits(i_layer, n_layers):
    """crates/llama/src/quant.rs:709-711"""
    return i_layer < n_layers // 8 or i_layer >= 7 * n_layers // 8 or (i_layer - n_layers // 8) % 3 == 2


def q4_k_m_type(name, n_layer):
    """The tensor types of a Q4_K_M file (crates/llama/src/quant.rs:786-1000): Q6_K for output.weight and
    for attn_v / ffn_down of the layers use_more_bits picks, Q4_K for the other matrices, F32 norms."""
    if name.endswith("_norm.weight"):
        return F32
    if name == "output.weight":
        return Q6_K
    if name.startswith("blk.") and (".attn_v." in name or ".ffn_down." in name):
        return Q6_K if use_more_bits(int(name.split(".")[1]), n_layer) else Q4_K
    return Q4_K


def tensor_shapes(hp):
    """{gguf name: (ne0, ne1)} of a llama-architecture model"""
    E, FF, V = hp["n_embd"], hp["n_ff"], hp["n_vocab"]
    EQ, EK = hp["n_head"] * hp["n_embd_head"], hp["n_head_kv"] * hp["n_embd_head"]
    shapes = {"token_embd.weight": (E, V), "output_norm.weight": (E, 1), "output.weight": (E, V)}
    for il in range(hp["n_layer"]):
        p = f"blk.{il}."
        shapes.update({p + "attn_norm.weight": (E, 1), p + "attn_q.weight": (E, EQ), p + "attn_k.weight": (E, EK),
                       p + "attn_v.weight": (E, EK), p + "attn_output.weight": (EQ, E), p + "ffn_norm.weight": (E, 1),
                       p + "ffn_gate.weight": (E, FF), p + "ffn_up.weight": (E, FF), p + "ffn_down.weight": (FF, E)})
    return shapes
