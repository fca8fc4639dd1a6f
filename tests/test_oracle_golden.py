"""The CPU oracle against the reference's golden vectors (bit-exact).

Every fixture under tests/golden/ was cut from a dump the reference commits
under parity/ (see tests/golden/extract_reference_vectors.py); the reference's
own tests replay the same dumps (crates/ggml/src/quants.rs:792, vec_dot.rs:2379
and :2798, repack.rs:5064/5689/6100, tiled.rs:1989, ops.rs:3154).
"""
import numpy as np
import pytest

import orc
from conftest import bits_equal

TY = {"Q4_0": orc.Q4_0, "Q8_0": orc.Q8_0, "Q4_K": orc.Q4_K, "Q6_K": orc.Q6_K, "Q8_K": orc.Q8_K, "MXFP4": orc.MXFP4}


def ref_input(n):
    """The LCG of parity/ref_quants_dump.c (crates/ggml/src/quants.rs:775-784)."""
    state = 0x12345678
    out = np.zeros(n, dtype=np.float32)
    for i in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        s = state - (1 << 32) if state >= (1 << 31) else state
        out[i] = np.float32(np.float32(np.float32(s) / np.float32(1 << 30)) * np.float32(0.75)) - np.float32(0.125)
    return out


def test_fp16_conversion(golden):
    g = golden("fp16cvt")
    x, want = g["x"], g["f16"]
    L = orc.lib()
    step = 7  # ~16k probes keep the scalar ctypes loop short
    got = np.array([L.orc_f32_to_f16(float(v)) for v in x[::step]], dtype=np.uint16)
    assert np.array_equal(got, want[::step])
    back = np.array([L.orc_f16_to_f32(int(h)) for h in range(0, 65536, 5)], dtype=np.float32)
    ref = np.arange(0, 65536, 5, dtype=np.uint16).view(np.float16).astype(np.float32)
    ok = (back.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(back) & np.isnan(ref))
    assert ok.all()


def test_weight_quantizers_and_dequantizers(golden):
    g = golden("quants")
    keys = sorted({k.rsplit("/", 1)[0] for k in g.files})
    seen = set()
    for key in keys:
        name, kind, n, _ = key.split("/")
        n = int(n)
        ty = TY[name]
        q, deq = g[key + "/q"], g[key + "/deq"]
        if kind == "sect":
            assert np.array_equal(orc.quantize(ty, ref_input(n)), q), f"{key}: quantized bytes"
        if deq.any():  # the Q8_K section carries no dequantized values
            assert bits_equal(orc.dequantize(ty, q, n), deq), f"{key}: dequantized values"
        seen.add(name)
    assert seen == {"Q4_0", "Q8_0", "Q4_K", "Q6_K", "Q8_K", "MXFP4"}


@pytest.mark.parametrize("tag", ["c3", "c1"])
@pytest.mark.parametrize("name", ["Q4_0", "Q8_0", "Q4_K", "Q6_K"])
def test_mul_mat_row_dot_route(golden, tag, name):
    """4 weight rows never qualify for the 8x8 layouts, so these pin the row-dot route."""
    g = golden("mulmat")
    W, X, dst = g[f"{tag}/{name}/W"], g[f"{tag}/{name}/X"], g[f"{tag}/{name}/dst"]
    out, route = orc.mul_mat(TY[name], W, X)
    assert route == orc.ROUTE_ROWDOT
    assert bits_equal(out, dst)


@pytest.mark.parametrize("name", ["Q4_K", "Q4_0", "MXFP4"])
def test_8x8_layout_activations_and_kernels(golden, name):
    g = golden("repack")
    ty = TY[name]
    n, nrows, nr_gemv, nr_gemm, nc = (int(v) for v in g[name + "/dims"])
    src, rep = g[name + "/src"], g[name + "/repacked"]
    assert np.array_equal(orc.repack_8x8(ty, src, nrows, n), rep)
    a1, a4 = g[name + "/gemv_act"], g[name + "/gemm_act"]
    if name == "Q4_K":
        assert np.array_equal(orc.quantize_q8_K(a1).ravel(), g[name + "/act_plain_q"])
        assert np.array_equal(orc.quantize_q8_K_4x8(a4), g[name + "/act_x4_q"])
    else:
        assert np.array_equal(orc.quantize_q8_0(a1).ravel(), g[name + "/act_plain_q"])
        assert np.array_equal(orc.quantize_q8_0_4x8(a4), g[name + "/act_x4_q"])
    assert bits_equal(orc.gemv_8x8(ty, n, rep, g[name + "/act_plain_q"], nc), g[name + "/gemv_out"])
    assert bits_equal(orc.gemm_8x8(ty, n, rep, g[name + "/act_x4_q"], nr_gemm, nc), g[name + "/gemm_out"])
    # the graph-level op picks the same route and reproduces both outputs
    W = src.reshape(nrows, -1)
    out, route = orc.mul_mat(ty, W, a4)
    assert route == orc.ROUTE_REPACK and bits_equal(out, g[name + "/gemm_out"])
    out, route = orc.mul_mat(ty, W, a1)
    assert route == orc.ROUTE_REPACK and bits_equal(out.ravel(), g[name + "/gemv_out"])


@pytest.mark.parametrize("key", ["q4k_goss", "q4k_granite", "q6k_granite", "q8_0_goss"])
def test_real_tensor_production_path(golden, key):
    g = golden("real_tensors")
    ty, n, rows, cols, flags = (int(v) for v in g[key + "/hdr"])
    W, act = g[key + "/W"], g[key + "/act"]
    out, route = orc.mul_mat(ty, W, act)
    if flags & 1:
        assert route == orc.ROUTE_REPACK
        assert bits_equal(out.ravel(), g[key + "/repack_out"])
        assert np.array_equal(orc.repack_8x8(ty, W, rows, n), g[key + "/repacked"])
    else:
        assert bits_equal(out, g[key + "/plain_out"])
    plain, _ = orc.mul_mat(ty, W, act, route=orc.ROUTE_ROWDOT)
    assert bits_equal(plain, g[key + "/plain_out"])
    q8k = g[key + "/q8k"]
    if q8k.size and n % 256 == 0:
        assert np.array_equal(orc.quantize_q8_K(act).ravel(), q8k)


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K"])
@pytest.mark.parametrize("shape", ["300x40", "300x12", "12x8", "188x300"])
def test_tiled_route(golden, name, shape):
    g = golden("tiled")
    key = f"mm/{name}/{shape}"
    out, route = orc.mul_mat(TY[name], g[key + "/W"], g[key + "/X"])
    assert route == orc.ROUTE_TILED
    assert bits_equal(out, g[key + "/dst"])


@pytest.mark.parametrize("name", ["Q4_K", "Q6_K"])
def test_mul_mat_id_tiled_and_row_dot_experts(golden, name):
    """5 experts, one of them with fewer than 8 routed rows (row-dot), the rest tiled."""
    g = golden("tiled")
    key = f"mmid/{name}"
    out, _ = orc.mul_mat_id(TY[name], g[key + "/W"], g[key + "/B"], g[key + "/ids"])
    assert bits_equal(out, g[key + "/dst"])
