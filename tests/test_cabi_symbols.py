"""The C-ABI library builds, loads without a GPU, and exports every function that
include/*.h declares."""
import ctypes
import glob
import os
import re

import b200

ROOT = b200.ROOT


def declared_functions():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        # function declarations: a name followed by '(' and terminated by ');' at statement level
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*(?:\([^()]*\)[^;{}()]*)*\)\s*;", text):
            name = m.group(1)
            if name.startswith(("b200_", "ggml_")) and not name.endswith("_t"):
                names.add(name)
    return names


def test_library_exports_every_declared_symbol():
    mod = b200.load()
    lib = ctypes.CDLL(mod.LIB_PATH)
    names = declared_functions()
    assert "b200_mul_mat" in names and "b200_flash_attn_ext" in names
    assert "ggml_build_forward_expand" in names and "ggml_backend_sched_graph_compute" in names and "ggml_time_us" in names
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, f"declared in include/ but not exported: {missing}"


def test_argument_errors_are_statuses_not_aborts():
    mod = b200.load()
    # unsupported weight type and bad k are refused before anything touches a device
    assert mod.lib.b200_weight_nbytes(mod.F32, 32, 256) == 0
    assert mod.lib.b200_weight_nbytes(mod.Q4_K, 32, 100) == 0
    assert mod.lib.b200_weight_nbytes(mod.Q4_K, 33, 256) == 2 * 4608
    rc = mod.lib.b200_mul_mat(mod.F32, 8, 256, 1, None, None, 256, None, 8, 0, None)
    assert rc == 3 and b"not supported" in mod.lib.b200_last_error()
    rc = mod.lib.b200_mul_mat(mod.Q4_K, 8, 100, 1, None, None, 100, None, 8, 0, None)
    assert rc == 3 and b"multiple of 256" in mod.lib.b200_last_error()


def test_prompt_kernel_choice_follows_cta_waves():
    """host arithmetic only: which Q4_K prompt kernel the library takes for (weight rows, activation rows) on 148 SMs"""
    lib = ctypes.CDLL(b200.load().LIB_PATH)
    f = lib.b200_prompt_kernel_choice
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
    # one wave of the integer kernel (128 x 32 per CTA) is never beaten by a kernel that first expands its operands
    assert f(4096, 64, 148) == 0 and f(4096, 128, 148) == 0 and f(1024, 512, 148) == 0
    # 192 CTAs of the integer kernel are two waves; 96 of the 64-column two-pass kernel are one
    assert f(4096, 192, 148) == 3 and f(4096, 256, 148) == 3
    # 512 activation rows on 4096 weight rows: 128 CTAs of the 128-column kernel are a single wave
    assert f(4096, 512, 148) == 4
    # ffn shapes at 512 rows: 448 CTAs x 1.6 against 896 CTAs: four long waves against seven short ones
    assert f(14336, 512, 148) == 4
    # a small GPU changes the wave counts, not the rule; sm_count <= 0 means 148
    assert f(4096, 64, 16) in (3, 4) and f(4096, 512, 0) == 4


def test_rows_add_fusable_is_host_arithmetic():
    """which (weight type, weight rows, activation rows) the few-rows kernels take with the residual add inside: 8 to 31 rows,
    Q4_K on the 8x8 route with whole groups of four rows, or Q6_K on the tiled route; answered without a device"""
    mod = b200.load()
    f = mod.lib.b200_mul_mat_q8_rows_add_fusable
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_int, ctypes.c_int64, ctypes.c_int64]
    assert f(mod.Q4_K, 4096, 16) == 1 and f(mod.Q4_K, 4096, 8) == 1 and f(mod.Q4_K, 4096, 28) == 1
    assert f(mod.Q4_K, 4096, 18) == 0          # two tail rows would go to another chain
    assert f(mod.Q4_K, 4100, 16) == 0          # rows not a multiple of 8: not the 8x8 route
    assert f(mod.Q6_K, 4096, 9) == 1 and f(mod.Q6_K, 100, 31) == 1
    assert f(mod.Q6_K, 4096, 7) == 0 and f(mod.Q6_K, 4096, 32) == 0 and f(mod.Q4_K, 4096, 1) == 0
    assert f(mod.Q8_0, 4096, 16) == 0 and f(mod.F32, 4096, 16) == 0 and f(mod.Q4_K, 0, 16) == 0


def test_rows_add_refuses_bad_arguments_before_touching_a_device():
    mod = b200.load()
    f = mod.lib.b200_mul_mat_q8_rows_add
    f.restype = ctypes.c_int
    i64, vp = ctypes.c_int64, ctypes.c_void_p
    f.argtypes = [ctypes.c_int, i64, i64, i64, vp, vp, ctypes.c_int, vp, i64, vp, i64, vp, i64, vp]
    one = 256
    # a weight type outside the path's five, a row length that is not a multiple of 256
    assert f(mod.F32, 4096, 4096, 16, one, one, mod.ACT_Q8_K_MIXED, one, 4096, one, 4096, one, 4096, None) != 0
    assert f(mod.Q4_K, 4096, 4000, 16, one, one, mod.ACT_Q8_K_MIXED, one, 4096, one, 4096, one, 4096, None) != 0
    # null pointers, row strides smaller than the rows
    assert f(mod.Q4_K, 4096, 4096, 16, one, one, mod.ACT_Q8_K_MIXED, one, 4096, None, 4096, one, 4096, None) != 0
    assert b"null pointer" in mod.lib.b200_last_error()
    assert f(mod.Q4_K, 4096, 4096, 16, one, one, mod.ACT_Q8_K_MIXED, one, 4096, one, 4000, one, 4096, None) != 0
    assert b"row strides" in mod.lib.b200_last_error()
    # a shape the few-rows kernels do not take, the wrong activation quantizer for the route
    assert f(mod.Q4_K, 4096, 4096, 64, one, one, mod.ACT_Q8_K_MIXED, one, 4096, one, 4096, one, 4096, None) != 0
    assert b"few-rows kernel" in mod.lib.b200_last_error()
    assert f(mod.Q4_K, 4096, 4096, 16, one, one, mod.ACT_Q8_K, one, 4096, one, 4096, one, 4096, None) != 0
    assert b"activation kind" in mod.lib.b200_last_error()
    # nothing to do
    assert f(mod.Q4_K, 0, 4096, 16, one, one, mod.ACT_Q8_K_MIXED, one, 4096, one, 4096, one, 4096, None) == 0
