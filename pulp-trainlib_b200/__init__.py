"""pulp-trainlib_b200: host-side mirror of the PULP-TrainLib C interface over libtrainlib_b200.so.

The product is the C-ABI shared library built from ``csrc/`` (hand-written CUDA for sm_100a).
This module only loads it through ctypes and offers small helpers to fill the reference's
argument structs from numpy arrays or device pointers.  There is no CPU fallback: loading
fails loudly when the library has not been built.
"""
import ctypes
import os

import numpy as np

from . import abi
from .abi import STRUCTS, FUNCTIONS, addr

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtrainlib_b200.so")

TL_OK = 0
TL_MEM_AUTO, TL_MEM_DEVICE, TL_MEM_HOST = 0, 1, 2
STEP_FW, STEP_WGT_GRAD, STEP_IN_GRAD = 0, 1, 2
LAYER_CONV2D, LAYER_DW_CONV, LAYER_PW_CONV, LAYER_LINEAR = 0, 1, 2, 3


def bind(lib, names=FUNCTIONS):
    """Give every `void f(void *)` entry point its ctypes signature."""
    for name in names:
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.argtypes = [ctypes.c_void_p]
        fn.restype = None
    return lib


_lib = None


def load(path=LIB_PATH):
    """Load libtrainlib_b200.so (once).  Raises if it is missing: nothing here computes on the CPU."""
    global _lib
    if _lib is not None and path == LIB_PATH:
        return _lib
    if not os.path.exists(path):
        raise RuntimeError("%s not found: build it with `make -C %s` (or __graft_entry__.build())"
                           % (path, os.path.join(_HERE, "csrc")))
    lib = bind(ctypes.CDLL(path))
    lib.trainlib_init.argtypes = [ctypes.c_int]; lib.trainlib_init.restype = ctypes.c_int
    lib.trainlib_last_error.restype = ctypes.c_int
    lib.trainlib_last_error_string.restype = ctypes.c_char_p
    lib.trainlib_malloc.argtypes = [ctypes.c_size_t]; lib.trainlib_malloc.restype = ctypes.c_void_p
    lib.trainlib_free.argtypes = [ctypes.c_void_p]
    lib.trainlib_malloc_host.argtypes = [ctypes.c_size_t]; lib.trainlib_malloc_host.restype = ctypes.c_void_p
    lib.trainlib_free_host.argtypes = [ctypes.c_void_p]
    lib.trainlib_memcpy_h2d.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]; lib.trainlib_memcpy_h2d.restype = ctypes.c_int
    lib.trainlib_memcpy_d2h.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]; lib.trainlib_memcpy_d2h.restype = ctypes.c_int
    lib.trainlib_memset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]; lib.trainlib_memset.restype = ctypes.c_int
    lib.trainlib_set_stream.argtypes = [ctypes.c_void_p]
    lib.trainlib_stream.restype = ctypes.c_void_p
    lib.trainlib_set_memory_mode.argtypes = [ctypes.c_int]
    lib.trainlib_memory_mode.restype = ctypes.c_int
    lib.trainlib_set_streams.argtypes = [ctypes.c_int]
    lib.trainlib_streams.restype = ctypes.c_int
    lib.trainlib_timer_stop_ms.restype = ctypes.c_double
    lib.trainlib_kernel_launches.restype = ctypes.c_longlong
    lib.trainlib_profile.argtypes = [ctypes.c_int]
    lib.trainlib_profile_entries.restype = ctypes.c_int
    lib.trainlib_profile_entry.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_double)]
    lib.trainlib_profile_entry.restype = ctypes.c_char_p
    lib.trainlib_profile_entry_flops.argtypes = [ctypes.c_int]
    lib.trainlib_profile_entry_flops.restype = ctypes.c_double
    lib.trainlib_graph_begin.restype = ctypes.c_int
    lib.trainlib_graph_end.restype = ctypes.c_void_p
    lib.trainlib_graph_launch.argtypes = [ctypes.c_void_p]; lib.trainlib_graph_launch.restype = ctypes.c_int
    lib.trainlib_graph_destroy.argtypes = [ctypes.c_void_p]
    lib.trainlib_memcpy_h2d_overlapped.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]; lib.trainlib_memcpy_h2d_overlapped.restype = ctypes.c_int
    lib.trainlib_mark_consumed.argtypes = [ctypes.c_int]; lib.trainlib_mark_consumed.restype = ctypes.c_int
    lib.trainlib_set_gemm_path.argtypes = [ctypes.c_int]
    lib.trainlib_gemm_path.restype = ctypes.c_int
    lib.trainlib_tc_status.restype = ctypes.c_int
    lib.trainlib_linear_fp32_bw_input_grads_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.trainlib_linear_fp32_bw_input_grads_noalloc.restype = ctypes.c_int
    lib.fastexp_gist.argtypes = [ctypes.c_float]; lib.fastexp_gist.restype = ctypes.c_float
    lib.q_rsqrt.argtypes = [ctypes.c_float]; lib.q_rsqrt.restype = ctypes.c_float
    if path == LIB_PATH:
        _lib = lib
    return lib


def check(lib):
    """Raise if the library has latched an error."""
    code = lib.trainlib_last_error()
    if code != TL_OK:
        msg = lib.trainlib_last_error_string().decode()
        lib.trainlib_clear_error()
        raise RuntimeError("trainlib_b200 error %d: %s" % (code, msg))


# ----------------------------------------------------------------------------- struct helpers
class Keep(object):
    """Owns the ctypes structs and arrays an argument struct points to (keeps them alive)."""

    def __init__(self):
        self.refs = []

    def hold(self, obj):
        self.refs.append(obj)
        return obj


def make_blob(keep, data=None, diff=None, C=1, H=1, W=1, dim=None, half=False):
    """struct blob / blob_fp16 over numpy arrays or device addresses."""
    cls = STRUCTS["blob_fp16" if half else "blob"]
    b = cls()
    b.data = addr(keep.hold(data)) if data is not None else None
    b.diff = addr(keep.hold(diff)) if diff is not None else None
    b.C, b.H, b.W = int(C), int(H), int(W)
    b.dim = int(dim if dim is not None else C * H * W)
    return keep.hold(b)


def make_args(keep, struct_name, **fields):
    """Fill one of the reference's argument structs; pointer fields accept structs, arrays, ints."""
    s = STRUCTS[struct_name]()
    kinds = dict(abi.STRUCT_FIELDS[struct_name])
    for k, v in fields.items():
        if k not in kinds:
            raise KeyError("%s has no field %s" % (struct_name, k))
        if kinds[k] == "ptr":
            setattr(s, k, addr(keep.hold(v)) if v is not None else None)
        elif kinds[k] == "fp16":
            setattr(s, k, int(np.float16(v).view(np.uint16)))
        else:
            setattr(s, k, v)
    return keep.hold(s)


def call(lib, name, args):
    getattr(lib, name)(ctypes.byref(args))


def profile_table(lib, flops=False):
    """[(kernel name, launches, total ms)] gathered since trainlib_profile(1), longest first; with flops=True a fourth
    field holds the useful floating-point operations the convolution kernels of that entry were launched for."""
    rows = []
    for i in range(lib.trainlib_profile_entries()):
        n = ctypes.c_longlong(0); ms = ctypes.c_double(0.0)
        name = lib.trainlib_profile_entry(i, ctypes.byref(n), ctypes.byref(ms))
        row = (name.decode(), int(n.value), float(ms.value))
        rows.append(row + (float(lib.trainlib_profile_entry_flops(i)),) if flops else row)
    return sorted(rows, key=lambda r: -r[2])


class DeviceBuffer(object):
    """A device allocation owned by Python, for resident-mode calls."""

    def __init__(self, lib, array=None, nbytes=None):
        self.lib = lib
        self.nbytes = int(array.nbytes if array is not None else nbytes)
        self.ptr = lib.trainlib_malloc(max(self.nbytes, 1))
        if not self.ptr:
            check(lib)
            raise MemoryError("trainlib_malloc(%d) failed" % self.nbytes)
        if array is not None:
            self.upload(array)

    def upload(self, array):
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        if self.lib.trainlib_memcpy_h2d(self.ptr, a.ctypes.data, a.nbytes) != TL_OK:
            check(self.lib)

    def download(self, dtype, shape):
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes
        if self.lib.trainlib_memcpy_d2h(out.ctypes.data, self.ptr, out.nbytes) != TL_OK:
            check(self.lib)
        return out

    def zero(self):
        self.lib.trainlib_memset(self.ptr, 0, self.nbytes)

    def free(self):
        if self.ptr:
            self.lib.trainlib_free(self.ptr)
            self.ptr = None
