"""A stand-in for the reference's registry and scheduler: loads libggml-b200.so the way
crates/ggml/src/backend.rs:1354-1416 does (dlopen, ggml_backend_init, api_version check) and
drives the vtables of include/ggml_b200_backend.h with ctypes (tensor mirror: sysffi.rs:208-227)."""
import ctypes as C

import numpy as np

F32, F16, I32 = 0, 1, 26
OP_NONE, OP_ADD, OP_MUL_MAT, OP_MUL_MAT_ID, OP_FLASH_ATTN_EXT, OP_VIEW = 0, 2, 29, 30, 74, 37
TYPE_TRAITS = {0: (1, 4), 1: (1, 2), 2: (32, 18), 8: (32, 34), 12: (256, 144), 14: (256, 210), 26: (1, 4), 27: (1, 8),
               39: (32, 17)}

vp, sz = C.c_void_p, C.c_size_t


class Tensor(C.Structure):
    pass


Tensor._fields_ = [
    ("type", C.c_int32), ("buffer", vp), ("ne", C.c_int64 * 4), ("nb", sz * 4), ("op", C.c_int32),
    ("op_params", C.c_int32 * 16), ("flags", C.c_int32), ("src", C.POINTER(Tensor) * 10),
    ("view_src", C.POINTER(Tensor)), ("view_offs", sz), ("data", vp), ("name", C.c_char * 64), ("extra", vp),
    ("padding", C.c_char * 8),
]
assert C.sizeof(Tensor) == 336


class Cgraph(C.Structure):
    _fields_ = [("size", C.c_int), ("n_nodes", C.c_int), ("n_leafs", C.c_int), ("nodes", C.POINTER(C.POINTER(Tensor))),
                ("grads", vp), ("grad_accs", vp), ("leafs", vp)]


def fn(res, *args):
    return C.CFUNCTYPE(res, *args)


class BufferTypeI(C.Structure):
    _fields_ = [("get_name", fn(C.c_char_p, vp)), ("alloc_buffer", fn(vp, vp, sz)), ("get_alignment", fn(sz, vp)),
                ("get_max_size", fn(sz, vp)), ("get_alloc_size", fn(sz, vp, C.POINTER(Tensor))), ("is_host", fn(C.c_bool, vp))]


class BufferType(C.Structure):
    _fields_ = [("iface", BufferTypeI), ("device", vp), ("context", vp)]


class BufferI(C.Structure):
    _fields_ = [("free_buffer", fn(None, vp)), ("get_base", fn(vp, vp)), ("init_tensor", fn(C.c_int, vp, C.POINTER(Tensor))),
                ("memset_tensor", fn(None, vp, C.POINTER(Tensor), C.c_uint8, sz, sz)),
                ("set_tensor", fn(None, vp, C.POINTER(Tensor), vp, sz, sz)),
                ("get_tensor", fn(None, vp, C.POINTER(Tensor), vp, sz, sz)),
                ("set_tensor_2d", vp), ("get_tensor_2d", vp),
                ("cpy_tensor", fn(C.c_bool, vp, C.POINTER(Tensor), C.POINTER(Tensor))), ("clear", fn(None, vp, C.c_uint8)),
                ("reset", vp)]


class Buffer(C.Structure):
    _fields_ = [("iface", BufferI), ("buft", vp), ("context", vp), ("size", sz), ("usage", C.c_int)]


class BackendI(C.Structure):
    _fields_ = [("get_name", fn(C.c_char_p, vp)), ("free", fn(None, vp)), ("set_tensor_async", vp), ("get_tensor_async", vp),
                ("cpy_tensor_async", vp), ("synchronize", fn(None, vp)), ("graph_plan_create", vp), ("graph_plan_free", vp),
                ("graph_plan_update", vp), ("graph_plan_compute", vp), ("graph_compute", fn(C.c_int, vp, C.POINTER(Cgraph))),
                ("event_record", vp), ("event_wait", vp), ("graph_optimize", vp)]


class Backend(C.Structure):
    _fields_ = [("guid", vp), ("iface", BackendI), ("device", vp), ("context", vp)]


class DevProps(C.Structure):
    _fields_ = [("name", C.c_char_p), ("description", C.c_char_p), ("memory_free", sz), ("memory_total", sz), ("type", C.c_int),
                ("device_id", C.c_char_p), ("caps", C.c_bool * 5)]


class DeviceI(C.Structure):
    _fields_ = [("get_name", fn(C.c_char_p, vp)), ("get_description", fn(C.c_char_p, vp)),
                ("get_memory", fn(None, vp, C.POINTER(sz), C.POINTER(sz))), ("get_type", fn(C.c_int, vp)),
                ("get_props", fn(None, vp, C.POINTER(DevProps))), ("init_backend", fn(vp, vp, C.c_char_p)),
                ("get_buffer_type", fn(vp, vp)), ("get_host_buffer_type", vp), ("buffer_from_host_ptr", vp),
                ("supports_op", fn(C.c_bool, vp, C.POINTER(Tensor))), ("supports_buft", fn(C.c_bool, vp, vp)),
                ("offload_op", fn(C.c_bool, vp, C.POINTER(Tensor))), ("event_new", vp), ("event_free", vp),
                ("event_synchronize", vp)]


class Device(C.Structure):
    _fields_ = [("iface", DeviceI), ("reg", vp), ("context", vp)]


class RegI(C.Structure):
    _fields_ = [("get_name", fn(C.c_char_p, vp)), ("get_device_count", fn(sz, vp)), ("get_device", fn(vp, vp, sz)),
                ("get_proc_address", fn(vp, vp, C.c_char_p))]


class Reg(C.Structure):
    _fields_ = [("api_version", C.c_int), ("iface", RegI), ("context", vp)]


def load_backend(path):
    """dlopen + ggml_backend_init, rejecting anything but api_version 2 (backend.rs:1390-1400)."""
    lib = C.CDLL(path)
    lib.ggml_backend_init.restype = C.POINTER(Reg)
    lib.ggml_backend_score.restype = C.c_int
    reg = lib.ggml_backend_init()
    if not reg or reg.contents.api_version != 2:
        raise RuntimeError("backend rejected: api_version != 2")
    return lib, reg


class Session:
    """One device, one backend, one buffer; tensors are laid out back to back like ggml-alloc would."""

    def __init__(self, lib, reg, device_index=0, buffer_bytes=1 << 28, params=None):
        self.lib, self.reg = lib, reg
        self.regp = C.cast(reg, vp)
        dev = reg.contents.iface.get_device(self.regp, device_index)
        assert dev, "no such device"
        self.devp = dev
        self.dev = C.cast(dev, C.POINTER(Device)).contents
        be = self.dev.iface.init_backend(dev, params)
        assert be, "init_backend failed"
        self.bep = be
        self.be = C.cast(be, C.POINTER(Backend)).contents
        self.buftp = self.dev.iface.get_buffer_type(dev)
        self.buft = C.cast(self.buftp, C.POINTER(BufferType)).contents
        self.bufp = self.buft.iface.alloc_buffer(self.buftp, buffer_bytes)
        assert self.bufp, "alloc_buffer failed"
        self.buf = C.cast(self.bufp, C.POINTER(Buffer)).contents
        self.base = self.buf.iface.get_base(self.bufp)
        self.align = self.buft.iface.get_alignment(self.buftp)
        self.offset = 0
        self.keep = []

    def close(self):
        self.be.iface.free(self.bep)
        self.buf.iface.free_buffer(self.bufp)

    def new_tensor(self, ty, ne, name=b"t", alloc=True):
        t = Tensor()
        t.type = ty
        ne = list(ne) + [1] * (4 - len(ne))
        blck, tsz = TYPE_TRAITS[ty]
        nb = [tsz, ne[0] // blck * tsz, 0, 0]
        nb[2] = nb[1] * ne[1]
        nb[3] = nb[2] * ne[2]
        for i in range(4):
            t.ne[i], t.nb[i] = ne[i], nb[i]
        t.name = name
        if alloc:
            need = self.buft.iface.get_alloc_size(self.buftp, C.byref(t))
            self.offset = (self.offset + self.align - 1) // self.align * self.align
            assert self.offset + need <= self.buf.size, "test buffer too small"
            t.buffer = self.bufp
            t.data = self.base + self.offset
            self.offset += need
            assert self.buf.iface.init_tensor(self.bufp, C.byref(t)) == 0
        self.keep.append(t)
        return t

    def set(self, t, arr):
        arr = np.ascontiguousarray(arr)
        self.buf.iface.set_tensor(self.bufp, C.byref(t), arr.ctypes.data, 0, arr.nbytes)

    def get(self, t, dtype, count):
        out = np.empty(count, dtype=dtype)
        self.buf.iface.get_tensor(self.bufp, C.byref(t), out.ctypes.data, 0, out.nbytes)
        return out

    def supports(self, t):
        return bool(self.dev.iface.supports_op(self.devp, C.byref(t)))

    def compute(self, nodes):
        arr = (C.POINTER(Tensor) * len(nodes))(*[C.pointer(n) for n in nodes])
        g = Cgraph()
        g.size = g.n_nodes = len(nodes)
        g.n_leafs = 0
        g.nodes = arr
        rc = self.be.iface.graph_compute(self.bep, C.byref(g))
        self.be.iface.synchronize(self.bep)
        return rc

    def last_error(self):
        self.lib.b200_last_error.restype = C.c_char_p
        return self.lib.b200_last_error().decode()
