"""ctypes binding of libdsqg_b200.so -- the C ABI declared in include/dsqg_b200.h.

The library is the only compute path of this package: if it is missing or cannot be
loaded, importing the binding raises.  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_size_t, c_void_p, POINTER

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libdsqg_b200.so")

DSQG_DTYPE_BF16 = 0
DSQG_DTYPE_F32 = 1
DSQG_MAX_TAPS = 128
DSQG_STATIC_SCRATCH_BYTES = 8 << 20

class Strides(ctypes.Structure):
    """dsqg_strides: element strides of the batch, head and row index."""
    _fields_ = [("batch", ctypes.c_longlong), ("head", ctypes.c_longlong), ("row", ctypes.c_longlong)]


# Every symbol include/dsqg_b200.h declares, with its ctypes signature.
_SIGNATURES = {
    "dsqg_status_str": (c_char_p, [c_int]),
    "dsqg_last_cuda_error": (c_char_p, []),
    "dsqg_version": (c_int, []),
    "dsqg_set_kernel_path": (c_int, [c_int]),
    "dsqg_device_error": (c_int, [c_int]),
    "dsqg_test_wait_timeout": (c_int, [ctypes.c_longlong, c_void_p]),
    "dsqg_fwd": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 2
                 + [c_int] * 5 + [c_void_p]),
    "dsqg_bwd_scratch_bytes": (c_size_t, [c_int] * 6),
    "dsqg_bwd": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 3
                 + [c_void_p] * 3 + [c_void_p] * 3 + [c_void_p, c_size_t] + [c_int] * 5 + [c_void_p]),
    "dsqg_tensor_core_path": (c_int, [c_int, c_int, POINTER(c_int32), c_int, c_int]),
    "dsqg_fwd_scaled": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 2
                        + [c_int] * 5 + [c_void_p, c_float]),
    "dsqg_bwd_scaled": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 3
                        + [c_void_p] * 3 + [c_void_p] * 3 + [c_void_p, c_size_t] + [c_int] * 5
                        + [c_void_p, c_float]),
    "dsqg_fwd_strided": (c_int, [c_void_p] * 3 + [POINTER(Strides)] + [c_void_p] * 2 + [POINTER(c_int32), c_int]
                         + [c_void_p, POINTER(Strides), c_void_p, c_void_p] + [c_int] * 5 + [c_void_p, c_float]),
    "dsqg_bwd_strided": (c_int, [c_void_p] * 3 + [POINTER(Strides)] + [c_void_p] * 2 + [POINTER(c_int32), c_int]
                         + [c_void_p] * 3 + [POINTER(Strides), c_void_p] + [c_void_p] * 5 + [c_void_p, c_size_t]
                         + [c_int] * 5 + [c_void_p, c_float]),
    "dsqg_fwd_strided_se": (c_int, [c_void_p] * 3 + [POINTER(Strides)] + [c_void_p] * 3 + [POINTER(c_int32), c_int]
                            + [c_void_p, POINTER(Strides), c_void_p, c_void_p] + [c_int] * 5 + [c_void_p, c_float]),
    "dsqg_bwd_strided_se": (c_int, [c_void_p] * 3 + [POINTER(Strides)] + [c_void_p] * 3 + [POINTER(c_int32), c_int]
                            + [c_void_p] * 3 + [POINTER(Strides), c_void_p] + [c_void_p] * 6 + [c_void_p, c_size_t]
                            + [c_int] * 5 + [c_void_p, c_float]),
    "dsqg_gate_bwd": (c_int, [c_void_p] * 3 + [POINTER(Strides)] + [c_void_p] * 3 + [c_int] * 4 + [c_void_p]),
    "dsqg_bwd_stages": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 3
                        + [c_void_p] * 3 + [c_void_p] * 3 + [c_void_p, c_size_t] + [c_int] * 5
                        + [c_void_p, c_int]),
    "dsqg_bwd_static": (c_int, [c_void_p] * 3 + [c_void_p] * 3 + [POINTER(c_int32), c_int] + [c_void_p] * 3
                        + [c_void_p] * 3 + [c_void_p] * 3 + [c_int] * 5 + [c_void_p]),
    "dsqg_ring_prefill": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_void_p]),
    "dsqg_decode": (c_int, [c_void_p] * 3 + [c_void_p] * 2 + [c_void_p] * 2 + [c_void_p] * 3
                    + [POINTER(c_int32), c_int, c_int] + [c_void_p] + [c_int] * 4 + [c_void_p]),
    "dsqg_causal_mean": (c_int, [c_void_p, c_void_p] + [c_int] * 5 + [c_void_p]),
    "dsqg_decode_kv": (c_int, [c_void_p] * 3 + [c_void_p] + [c_void_p] * 2 + [c_void_p] * 3
                       + [POINTER(c_int32), c_int, c_int] + [c_void_p] + [c_int] * 4 + [c_void_p, c_int]),
    "dsqg_ring_prefill_kv": (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_void_p]),
    "dsqg_decode_overlapped": (c_int, [c_void_p] * 3 + [c_void_p] * 2 + [c_void_p] * 2 + [c_void_p] * 3
                               + [POINTER(c_int32), c_int, c_int] + [c_void_p] + [c_int] * 4 + [c_void_p]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


class DSQGError(RuntimeError):
    """Raised when the native library reports a non-zero status."""

    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        msg = f"{where} failed with status {status}: {detail}"
        super().__init__(msg)


_lib = None


def load():
    """Load libdsqg_b200.so (once) and attach argument types.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m dwarf_b200.build` "
            "(needs nvcc; targets sm_100a). dwarf_b200 has no fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int, where: str):
    if status != 0:
        lib = load()
        detail = lib.dsqg_status_str(status).decode()
        if status == -7:
            detail += " -- " + lib.dsqg_last_cuda_error().decode()
        raise DSQGError(status, where, detail)


_offset_cache = {}


def offsets_array(offsets):
    """Host int32 array for an offsets tuple (cached; the ABI takes a host pointer)."""
    key = tuple(int(o) for o in offsets)
    arr = _offset_cache.get(key)
    if arr is None:
        arr = (c_int32 * len(key))(*key)
        _offset_cache[key] = arr
    return arr, len(key)
