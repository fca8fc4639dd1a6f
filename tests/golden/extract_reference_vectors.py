#!/usr/bin/env python3
"""Extract the hot-path golden vectors from the reference's committed dumps.

The reference keeps bit-exact dumps of the original C implementation under its
`parity/` directory (formats documented in parity/ref_*_dump.c*).  This script
copies out only the sections that pin the quantized mat-mul / flash-attention
path (Q4_0, Q8_0, Q4_K, Q6_K, MXFP4, Q8_K; F16-KV attention) into compact
`.npz` files next to this script, so the tests run where the reference tree is
not available.

    python tests/golden/extract_reference_vectors.py <reference_root>

Outputs: quants.npz, mulmat.npz, repack.npz, real_tensors.npz, tiled.npz,
fp16cvt.npz, flash_attn.npz, flash_attn_probe.npz.
"""
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
HOT_TYPES = {2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K", 15: "Q8_K", 39: "MXFP4"}
# bytes per block / elements per block for every type id the dumps contain
BLOCK = {1: (2, 1), 30: (2, 1), 2: (18, 32), 3: (20, 32), 6: (22, 32), 7: (24, 32), 8: (34, 32), 9: (36, 32),
         10: (84, 256), 11: (110, 256), 12: (144, 256), 13: (176, 256), 14: (210, 256), 15: (292, 256),
         16: (66, 256), 17: (74, 256), 18: (98, 256), 19: (50, 256), 21: (110, 256), 22: (82, 256),
         23: (136, 256), 29: (56, 256), 39: (17, 32), 40: (36, 64)}


def row_size(ty, n):
    b, e = BLOCK[ty]
    return n // e * b


def u8(b):
    return np.frombuffer(b, dtype=np.uint8).copy()


def f32(b):
    return np.frombuffer(b, dtype=np.float32).copy()


def len_sections(path):
    b = open(path, "rb").read()
    o, out = 0, []
    while o < len(b):
        (n,) = struct.unpack_from("<I", b, o)
        out.append(b[o + 4:o + 4 + n])
        o += 4 + n
    return out


def extract_quants(par, out):
    """parity/quants_ref.bin and quants_ref_fp4.bin (format: parity/ref_quants_dump.c:4-7)."""
    for fn in ("quants_ref.bin", "quants_ref_fp4.bin"):
        b = open(os.path.join(par, fn), "rb").read()
        o, idx = 0, 0
        while True:
            (magic,) = struct.unpack_from("<I", b, o)
            if magic == 0xFFFF:
                break
            ty, n, qlen = struct.unpack_from("<IQQ", b, o + 4)
            q = b[o + 24:o + 24 + qlen]
            d = b[o + 24 + qlen:o + 24 + qlen + 4 * n]
            o += 24 + qlen + 4 * n
            if ty in HOT_TYPES:
                kind = "sect" if magic == 0x54434553 else "raw"
                key = f"{HOT_TYPES[ty]}/{kind}/{n}/{idx}"
                out[key + "/q"] = u8(q)
                out[key + "/deq"] = f32(d)
                idx += 1


def extract_mulmat(par, out):
    """parity/mulmat_ref.bin (ne11 = 3) and mulmat_ref_c1.bin (ne11 = 1): parity/ref_mulmat_dump.c:5-7."""
    for fn, tag in (("mulmat_ref.bin", "c3"), ("mulmat_ref_c1.bin", "c1")):
        b = open(os.path.join(par, fn), "rb").read()
        o = 0
        while True:
            (magic,) = struct.unpack_from("<I", b, o)
            if magic == 0xFFFFFFFF:
                break
            assert magic == 0x314D4D56
            ty, n, R, C = struct.unpack_from("<IIII", b, o + 4)
            o += 20
            rs = row_size(ty, n)
            W = b[o:o + rs * R]
            o += rs * R
            X = b[o:o + 4 * n * C]
            o += 4 * n * C
            D = b[o:o + 4 * R * C]
            o += 4 * R * C
            if ty in HOT_TYPES:
                key = f"{tag}/{HOT_TYPES[ty]}"
                out[key + "/W"] = u8(W).reshape(R, rs)
                out[key + "/X"] = f32(X).reshape(C, n)
                out[key + "/dst"] = f32(D).reshape(C, R)


def extract_repack(par, out):
    """The three 8x8 dumps: parity/ref_repack_kdump.cpp:15-29, ref_repack_dump.cpp:16-28."""
    for fn, ty in (("q4k_repack_ref.bin", 12), ("q4_0_repack_ref.bin", 2), ("repack_ref.bin", 39)):
        s = len_sections(os.path.join(par, fn))
        h = struct.unpack("<6I", s[0])
        if ty == 39:
            n, nrows, nr_gemv, nr_gemm, nc, _ = h
        else:
            _, n, nrows, nr_gemv, nr_gemm, nc = h
        key = HOT_TYPES[ty]
        out[key + "/dims"] = np.array([n, nrows, nr_gemv, nr_gemm, nc], dtype=np.int64)
        out[key + "/src"] = u8(s[1])
        out[key + "/repacked"] = u8(s[2])
        out[key + "/act_plain_q"] = u8(s[3])
        out[key + "/act_x4_q"] = u8(s[4])
        out[key + "/gemv_out"] = f32(s[5])[:nc]
        out[key + "/gemm_out"] = f32(s[6])[:nr_gemm * nc].reshape(nr_gemm, nc)
        out[key + "/gemv_act"] = f32(s[9]).reshape(nr_gemv, n)
        out[key + "/gemm_act"] = f32(s[10]).reshape(nr_gemm, n)


def extract_real(par, out):
    """Real-GGUF tensor dumps (parser: crates/ggml/src/vec_dot.rs:2748-2775)."""
    for fn in ("q4k_goss_ref.bin", "q4k_granite_ref.bin", "q6k_granite_ref.bin", "q8_0_goss_ref.bin"):
        s = len_sections(os.path.join(par, fn))
        ty, n, rows, cols, flags, _ = struct.unpack("<6I", s[0])
        key = fn[:-8]
        out[key + "/hdr"] = np.array([ty, n, rows, cols, flags], dtype=np.int64)
        out[key + "/W"] = u8(s[1]).reshape(rows, -1)
        out[key + "/act"] = f32(s[2]).reshape(cols, n)
        out[key + "/plain_out"] = f32(s[3]).reshape(cols, rows)
        out[key + "/repacked"] = u8(s[4])
        out[key + "/repack_out"] = f32(s[5])
        out[key + "/q8k"] = u8(s[6])


def extract_tiled(par, out):
    """parity/tiled_ref.bin, Q4_K and Q6_K sections only (parity/ref_tiled_dump.c:19-27)."""
    b = open(os.path.join(par, "tiled_ref.bin"), "rb").read()
    o = 0
    while True:
        (magic,) = struct.unpack_from("<I", b, o)
        o += 4
        if magic == 0xFFFFFFFF:
            break
        assert magic == 0x31544D56
        kind, ty, n, R, C = struct.unpack_from("<5I", b, o)
        o += 20
        rs = row_size(ty, n)
        if kind == 0:
            W, o = b[o:o + rs * R], o + rs * R
            X, o = b[o:o + 4 * n * C], o + 4 * n * C
            D, o = b[o:o + 4 * R * C], o + 4 * R * C
            if ty in (12, 14):
                key = f"mm/{HOT_TYPES[ty]}/{R}x{C}"
                out[key + "/W"] = u8(W).reshape(R, rs)
                out[key + "/X"] = f32(X).reshape(C, n)
                out[key + "/dst"] = f32(D).reshape(C, R)
        else:
            n_as, n_ids, ne12 = struct.unpack_from("<3I", b, o)
            o += 12
            W, o = b[o:o + rs * R * n_as], o + rs * R * n_as
            Y, o = b[o:o + 4 * n * C * ne12], o + 4 * n * C * ne12
            I, o = b[o:o + 4 * n_ids * ne12], o + 4 * n_ids * ne12
            D, o = b[o:o + 4 * R * n_ids * ne12], o + 4 * R * n_ids * ne12
            if ty in (12, 14):
                key = f"mmid/{HOT_TYPES[ty]}"
                out[key + "/W"] = u8(W).reshape(n_as, R, rs)
                out[key + "/B"] = f32(Y).reshape(ne12, C, n)
                out[key + "/ids"] = np.frombuffer(I, dtype=np.int32).copy().reshape(ne12, n_ids)
                out[key + "/dst"] = f32(D).reshape(ne12, n_ids, R)


def extract_fp16cvt(par, out):
    """parity/fp16cvt_probe.bin (format: parity/ref_fp16cvt_probe.c:25-28)."""
    b = open(os.path.join(par, "fp16cvt_probe.bin"), "rb").read()
    magic, n = struct.unpack_from("<II", b, 0)
    assert magic == 0x43363146 and len(b) == 8 + n * 10
    bat = np.frombuffer(b, dtype=np.float32, count=n, offset=8)
    new = np.frombuffer(b, dtype=np.uint16, count=n, offset=8 + n * 6)  # the F16C bulk column
    # every 4th probe keeps the file small; NaN inputs are dropped because the
    # reference's own scalar and bulk paths disagree on NaN payloads
    keep = np.zeros(n, dtype=bool)
    keep[::4] = True
    keep &= ~np.isnan(bat)
    out["x"] = bat[keep].copy()
    out["f16"] = new[keep].copy()


def extract_flash_attn(par, out):
    """parity/fa_ref.bin: 15 cases x 8 length-prefixed sections (parity/ref_fa_dump.c:18-33).
    Only the cases whose K and V are both F16 are kept."""
    s = len_sections(os.path.join(par, "fa_ref.bin"))
    assert len(s) % 8 == 0
    kept = 0
    for c in range(len(s) // 8):
        sec = s[8 * c:8 * c + 8]
        hdr = np.frombuffer(sec[0], dtype=np.int64).copy()
        mode, dk, dv, h, h_kv, t, s_kv, kty, vty = hdr
        if kty != 1 or vty != 1:
            continue
        key = f"case{c}"
        out[key + "/hdr"] = hdr
        out[key + "/q"] = f32(sec[1])
        out[key + "/k"] = np.frombuffer(sec[2], dtype=np.uint16).copy()
        out[key + "/v"] = np.frombuffer(sec[3], dtype=np.uint16).copy()
        out[key + "/mask"] = np.frombuffer(sec[4], dtype=np.uint16).copy()
        out[key + "/sinks"] = f32(sec[5])
        out[key + "/dst"] = f32(sec[6])
        out[key + "/params"] = f32(sec[7])
        kept += 1
    out["n_cases"] = np.array([kept], dtype=np.int64)


def extract_flash_attn_probe(par, out):
    """parity/fa_probe.bin (format: parity/ref_fa_probe.c:18-24): per probe the inputs, then records
    (tag, t, nth, dst): tag 0 = the T-row run, 1 = the 1-row run of token t (split-KV from 512 KV
    positions on, with nth chunks), 2 = rows 1..T-1.  Kept: the two S_kv = 600 probes."""
    b = open(os.path.join(par, "fa_probe.bin"), "rb").read()
    o, n = 0, len(b)

    def sec():
        nonlocal o
        (ln,) = struct.unpack_from("<I", b, o)
        s = b[o + 4:o + 4 + ln]
        o += 4 + ln
        return s

    probe = -1
    keep = False
    while o < n:
        (tag,) = struct.unpack_from("<I", b, o)
        if tag == 0xF17E0001:
            o += 4
            probe += 1
            geom = np.frombuffer(sec(), dtype=np.int64).copy()
            knobs = f32(sec())
            q, k, v, m, s = sec(), sec(), sec(), sec(), sec()
            keep = int(geom[5]) >= 512
            if keep:
                key = f"probe{probe}"
                out[key + "/geom"] = geom
                out[key + "/knobs"] = knobs
                out[key + "/q"] = f32(q)
                out[key + "/k"] = np.frombuffer(k, dtype=np.uint16).copy()
                out[key + "/v"] = np.frombuffer(v, dtype=np.uint16).copy()
                out[key + "/mask"] = np.frombuffer(m, dtype=np.uint16).copy()
                out[key + "/sinks"] = f32(s)
            continue
        tag, t, nth = struct.unpack_from("<III", b, o)
        o += 12
        d = sec()
        if keep:
            out[f"probe{probe}/rec/{tag}/{t}/{nth}"] = f32(d)


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    par = os.path.join(sys.argv[1], "parity")
    for name, fn in (("quants", extract_quants), ("mulmat", extract_mulmat), ("repack", extract_repack),
                     ("real_tensors", extract_real), ("tiled", extract_tiled), ("fp16cvt", extract_fp16cvt),
                     ("flash_attn", extract_flash_attn), ("flash_attn_probe", extract_flash_attn_probe)):
        out = {}
        fn(par, out)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(f"{name}.npz: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
