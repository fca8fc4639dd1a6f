"""ctypes bindings of include/ggml_base_b200.h, shaped like the reference's CLibSyms (sysffi.rs:458-629):
every symbol resolved by name, tensors mirrored as in ggml_plugin.Tensor."""
import ctypes as C

import b200
from ggml_plugin import Cgraph, Tensor

vp, sz = C.c_void_p, C.c_size_t
TP = C.POINTER(Tensor)


class InitParams(C.Structure):
    _fields_ = [("mem_size", sz), ("mem_buffer", vp), ("no_alloc", C.c_bool)]


SIGNATURES = {
    "ggml_init": (vp, [InitParams]), "ggml_free": (None, [vp]), "ggml_new_tensor": (TP, [vp, C.c_int, C.c_int, C.POINTER(C.c_int64)]),
    "ggml_set_name": (TP, [TP, C.c_char_p]), "ggml_set_input": (None, [TP]), "ggml_set_output": (None, [TP]),
    "ggml_tensor_overhead": (sz, []), "ggml_graph_overhead_custom": (sz, [sz, C.c_bool]),
    "ggml_new_graph_custom": (C.POINTER(Cgraph), [vp, sz, C.c_bool]), "ggml_build_forward_expand": (None, [C.POINTER(Cgraph), TP]),
    "ggml_graph_n_nodes": (C.c_int, [C.POINTER(Cgraph)]), "ggml_graph_node": (TP, [C.POINTER(Cgraph), C.c_int]),
    "ggml_graph_nodes": (C.POINTER(TP), [C.POINTER(Cgraph)]),
    "ggml_backend_buft_alloc_buffer": (vp, [vp, sz]), "ggml_backend_buft_get_alignment": (sz, [vp]),
    "ggml_backend_buft_get_max_size": (sz, [vp]), "ggml_backend_buft_get_alloc_size": (sz, [vp, TP]),
    "ggml_backend_buffer_free": (None, [vp]), "ggml_backend_buffer_get_base": (vp, [vp]), "ggml_backend_buffer_clear": (None, [vp, C.c_uint8]),
    "ggml_backend_buffer_set_usage": (None, [vp, C.c_int]), "ggml_backend_tensor_set": (None, [TP, vp, sz, sz]),
    "ggml_backend_tensor_get": (None, [TP, vp, sz, sz]), "ggml_backend_tensor_alloc": (C.c_int, [vp, TP, vp]),
    "ggml_backend_view_init": (C.c_int, [TP]), "ggml_backend_cpu_buffer_from_ptr": (vp, [vp, sz]), "ggml_backend_cpu_buffer_type": (vp, []),
    "ggml_backend_dev_count": (sz, []), "ggml_backend_dev_get": (vp, [sz]), "ggml_backend_dev_by_name": (vp, [C.c_char_p]),
    "ggml_backend_dev_by_type": (vp, [C.c_int]), "ggml_backend_dev_name": (C.c_char_p, [vp]), "ggml_backend_free": (None, [vp]),
    "ggml_backend_dev_init": (vp, [vp, C.c_char_p]), "ggml_backend_dev_buffer_type": (vp, [vp]), "ggml_backend_dev_backend_reg": (vp, [vp]),
    "ggml_backend_reg_get_proc_address": (vp, [vp, C.c_char_p]), "ggml_backend_load_all_from_path": (None, [C.c_char_p]),
    "ggml_backend_sched_new": (vp, [C.POINTER(vp), C.POINTER(vp), C.c_int, sz, C.c_bool, C.c_bool]), "ggml_backend_sched_free": (None, [vp]),
    "ggml_backend_sched_reset": (None, [vp]), "ggml_backend_sched_alloc_graph": (C.c_bool, [vp, C.POINTER(Cgraph)]),
    "ggml_backend_sched_graph_compute": (C.c_int, [vp, C.POINTER(Cgraph)]), "ggml_backend_sched_synchronize": (None, [vp]),
    "ggml_backend_sched_set_tensor_backend": (None, [vp, TP, vp]), "ggml_backend_sched_get_tensor_backend": (vp, [vp, TP]),
    "ggml_backend_sched_get_n_backends": (C.c_int, [vp]), "ggml_backend_sched_get_backend": (vp, [vp, C.c_int]),
    "ggml_backend_sched_get_buffer_size": (sz, [vp, vp]), "ggml_time_us": (C.c_int64, []),
    "ggml_backend_synchronize": (None, [vp]), "ggml_backend_tensor_set_async": (None, [vp, TP, vp, sz, sz]),
    "ggml_backend_tensor_get_async": (None, [vp, TP, vp, sz, sz]),
    "ggml_backend_sched_set_copy_callback": (None, [vp, vp, vp]),
    "b200_gpu_layer_start": (sz, [sz, C.c_int32]), "b200_layer_on_gpu": (C.c_bool, [sz, C.c_int32, sz]),
}
# the names CLibSyms::resolve asks for (ggml_backend_time_us is resolved as "ggml_time_us")
CLIB_SYMS = [n for n in SIGNATURES if not n.startswith("b200_")]


def load():
    lib = C.CDLL(b200.load().LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        f = getattr(lib, name)
        f.restype, f.argtypes = res, args
    return lib


def new_tensor(lib, ctx, ty, ne, name=None):
    arr = (C.c_int64 * len(ne))(*ne)
    t = lib.ggml_new_tensor(ctx, ty, len(ne), arr)
    assert t, "ggml_new_tensor failed"
    if name:
        lib.ggml_set_name(t, name)
    return t


def op_node(lib, ctx, ty, ne, op, srcs, name=None, params=None):
    """what the reference's emitter does: a fresh tensor, then op / src / op_params written directly"""
    t = new_tensor(lib, ctx, ty, ne, name)
    t.contents.op = op
    for i, s in enumerate(srcs):
        t.contents.src[i] = s
    if params is not None:
        raw = bytes(params)
        C.memmove(t.contents.op_params, raw, len(raw))
    return t
