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
