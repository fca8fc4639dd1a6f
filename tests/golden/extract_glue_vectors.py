#!/usr/bin/env python3
"""Cuts glue-op golden vectors out of the reference's node dump of a synthetic decoder
(parity/qwen4exp_qsa_nodes_fa_ref.bin, written by parity/ref_decode_dump_noembd.c against the C
ggml build the reference is a port of; stream format "DECDMP1", parity/ref_decode_dump.c:32-47).

The stream holds every graph node's output but not the graph edges, so an op's inputs are taken
from the nodes just before it and kept only when a float64 numpy model of the op agrees to 1e-5;
the tests then demand bit equality from the oracle and from the CUDA kernels.

    python tests/golden/extract_glue_vectors.py /path/to/reference   ->  tests/golden/glue_nodes.npz

The synthetic model (crates/llama/tests/qwen4exp_qsa_dump.rs:306-345): rms eps 1e-5, rope over all
16 channels of a head with NEOX pairing and frequency base 10000, 2 prompt tokens at positions 0, 1
and 12 single-token steps after them.
"""
import struct
import sys
from pathlib import Path

import numpy as np

ELEM_CAP = 1 << 19
EPS = 1e-5


def parse(path):
    f = open(path, "rb")
    assert f.read(8) == b"DECDMP1\0"
    (n_tok,) = struct.unpack("<I", f.read(4))
    f.read(4 * n_tok)
    (n_nodes,) = struct.unpack("<I", f.read(4))
    nodes = []
    for _ in range(n_nodes):
        strs = []
        for _ in range(3):
            (ln,) = struct.unpack("<B", f.read(1))
            strs.append(f.read(ln).decode())
        ne = struct.unpack("<4q", f.read(32))
        (n,) = struct.unpack("<Q", f.read(8))
        e = np.frombuffer(f.read(4 * n), dtype=np.float32) if n < ELEM_CAP else None
        nodes.append(dict(op=strs[0], name=strs[1], ty=strs[2], ne=ne, n=n, e=e))
    return n_tok, nodes


def close(a, b):
    return a.shape == b.shape and np.allclose(a, b, rtol=1e-5, atol=1e-7)


def main():
    ref = Path(sys.argv[1])
    n_prompt, nodes = parse(ref / "parity" / "qwen4exp_qsa_nodes_fa_ref.bin")
    starts = [i for i, n in enumerate(nodes) if n["op"] == "GET_ROWS" and n["name"] == "model.input_embed"]
    out = {}
    count = {"rms_norm": 0, "silu": 0, "swiglu": 0, "add": 0, "rope": 0, "set_rows": 0}

    def pass_of(i):
        return sum(1 for s in starts[1:] if i >= s)

    for i, n in enumerate(nodes):
        if n["e"] is None or n["n"] == 0 or i == 0:
            continue
        p = pass_of(i)
        prev = nodes[i - 1]
        ne0 = n["ne"][0]
        if n["op"] == "RMS_NORM" and p < 3 and prev["e"] is not None and prev["n"] == n["n"]:
            x = prev["e"].astype(np.float64).reshape(-1, ne0)
            y = x / np.sqrt((x * x).mean(axis=1, keepdims=True) + EPS)
            if close(y.ravel(), n["e"].astype(np.float64)):
                k = count["rms_norm"]
                out[f"rms_norm_{k}_x"], out[f"rms_norm_{k}_y"] = prev["e"].reshape(-1, ne0), n["e"].reshape(-1, ne0)
                count["rms_norm"] += 1
        elif n["op"] == "SILU" and p < 3 and prev["e"] is not None and prev["n"] == n["n"]:
            x = prev["e"].astype(np.float64)
            if close(x / (1 + np.exp(-x)), n["e"].astype(np.float64)):
                k = count["silu"]
                out[f"silu_{k}_x"], out[f"silu_{k}_y"] = prev["e"].reshape(-1, ne0), n["e"].reshape(-1, ne0)
                count["silu"] += 1
        elif n["op"] == "SWIGLU" and p < 3 and i >= 2:
            g, u = nodes[i - 2], nodes[i - 1]
            if g["e"] is not None and u["e"] is not None and g["n"] == n["n"] == u["n"]:
                x = g["e"].astype(np.float64)
                if close(x / (1 + np.exp(-x)) * u["e"], n["e"].astype(np.float64)):
                    k = count["swiglu"]
                    out[f"swiglu_{k}_x"], out[f"swiglu_{k}_g"] = g["e"].reshape(-1, ne0), u["e"].reshape(-1, ne0)
                    out[f"swiglu_{k}_y"] = n["e"].reshape(-1, ne0)
                    count["swiglu"] += 1
        elif n["op"] == "ADD" and p < 3:
            # a + b with both operands among the six nodes before the sum
            found = False
            for ia in range(max(0, i - 6), i):
                for ib in range(ia + 1, i):
                    a, b = nodes[ia], nodes[ib]
                    if a["e"] is None or b["e"] is None or a["n"] != n["n"] or b["n"] != n["n"]:
                        continue
                    if np.array_equal((a["e"] + b["e"]).view(np.uint32), n["e"].view(np.uint32)) and np.any(a["e"]) and np.any(b["e"]):
                        k = count["add"]
                        out[f"add_{k}_a"], out[f"add_{k}_b"], out[f"add_{k}_y"] = a["e"], b["e"], n["e"]
                        count["add"] += 1
                        found = True
                        break
                if found:
                    break
        elif n["op"] == "ROPE" and n["name"].startswith(("Qcur", "Kcur")) and prev["n"] == n["n"]:
            pos = np.arange(n_prompt, dtype=np.int32) if p == 0 else np.array([n_prompt + p - 1], dtype=np.int32)
            ne = n["ne"]
            if ne[2] == len(pos):
                k = count["rope"]
                out[f"rope_{k}_x"] = prev["e"].reshape(ne[2], ne[1], ne[0])
                out[f"rope_{k}_y"] = n["e"].reshape(ne[2], ne[1], ne[0])
                out[f"rope_{k}_pos"] = pos
                count["rope"] += 1
        elif n["op"] == "SET_ROWS" and n["ty"] == "f16" and n["name"].startswith(("cache_k_l", "cache_v_l")) and p in (0, 1, 7):
            # the rows this pass wrote: source = the f32 view just before, destination rows = positions
            pos = np.arange(n_prompt, dtype=np.int64) if p == 0 else np.array([n_prompt + p - 1], dtype=np.int64)
            if prev["e"] is not None and prev["n"] == ne0 * len(pos):
                src = prev["e"].reshape(len(pos), ne0)
                dst = n["e"].reshape(-1, ne0)
                if np.allclose(dst[pos], src, rtol=2e-3, atol=1e-6):
                    k = count["set_rows"]
                    out[f"set_rows_{k}_x"], out[f"set_rows_{k}_idx"] = src, pos
                    out[f"set_rows_{k}_y"] = dst[pos].astype(np.float16)   # exact: the dump widened f16 to f32
                    count["set_rows"] += 1
    for k, v in count.items():
        out[f"n_{k}"] = np.int64(v)
    dest = Path(__file__).parent / "glue_nodes.npz"
    np.savez_compressed(dest, **out)
    print(count, dest, dest.stat().st_size)
    # the reference GGUF writer's golden file (parity/ref_gguf_write.c), taken as it is: 416 bytes
    gguf = Path(__file__).parent / "gguf_write_ref.bin"
    gguf.write_bytes((ref / "parity" / "gguf_write_ref.bin").read_bytes())
    print(gguf, gguf.stat().st_size)


if __name__ == "__main__":
    main()
