"""ctypes binding of the C ABI declared in include/dci_b200.h.

The CUDA library is the only implementation: if libdci_b200.so is missing this
module raises at import of the first symbol instead of falling back to anything.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdci_b200.so")

# every symbol include/dci_b200.h declares: (name, restype, argtypes)
_c_fp = C.POINTER(C.c_float)
_c_ip = C.POINTER(C.c_int)
_c_llp = C.POINTER(C.c_longlong)
_vp = C.c_void_p
SYMBOLS = [
    ("dci_b200_last_error", C.c_char_p, []),
    ("dci_b200_abi_version", C.c_int, []),
    ("dci_b200_create", C.c_int, [C.POINTER(_vp), C.c_int, C.c_int, C.c_int, C.c_int, C.c_ulonglong]),
    ("dci_b200_destroy", C.c_int, [_vp]),
    ("dci_b200_get_proj", C.c_int, [_vp, _vp]),
    ("dci_b200_set_proj", C.c_int, [_vp, _vp]),
    ("dci_b200_add", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    ("dci_b200_last_projection_ms", C.c_int, [_vp, C.POINTER(C.c_float)]),
    ("dci_b200_append", C.c_int, [_vp, _vp, C.c_int, _vp]),
    ("dci_b200_blind_width", C.c_int, [C.c_int, C.c_int]),
    ("dci_b200_query_blind", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    ("dci_b200_query", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                 _vp, _vp, _vp]),
    ("dci_b200_query_host", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_int, _vp, _vp]),
    ("dci_b200_clear", C.c_int, [_vp]),
    ("dci_b200_reset", C.c_int, [_vp, C.c_ulonglong]),
    ("dci_b200_num_points", C.c_int, [_vp]),
    ("dci_b200_get_index", C.c_int, [_vp, _vp, _vp]),
    ("dci_b200_set_index", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    ("dci_b200_project", C.c_int, [_vp, _vp, C.c_int, _vp, _vp]),
    ("dci_b200_enable_work_stats", C.c_int, [_vp, C.c_int]),
    ("dci_b200_get_work_stats", C.c_int, [_vp, _vp, C.c_longlong]),
    ("dci_b200_get_phase_cycles", C.c_int, [_vp, _vp]),
    ("dci_b200_launch_count", C.c_longlong, [_vp]),
    ("dci_b200_device_alloc_calls", C.c_longlong, []),
    ("dci_b200_set_max_ctas", C.c_int, [_vp, C.c_int]),
    ("dci_b200_set_projection", C.c_int, [_vp, C.c_int]),
    ("dci_b200_enable_timing", C.c_int, [_vp, C.c_int]),
    ("dci_b200_get_timing", C.c_int, [_vp, _vp]),
    ("dci_b200_query_noalloc", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                         _vp, _vp, _vp]),
    ("dci_b200_merge_shards", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _c_llp, _vp, _vp, C.c_int, _vp]),
    ("dci_b200_query_packed", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp]),
    ("dci_b200_merge_shards_packed", C.c_int, [_vp, C.c_int, C.c_int, C.c_int, _c_llp, _vp, _vp, C.c_int, _vp]),
    ("dci_b200_mdci_create", C.c_int, [C.POINTER(_vp), C.c_int, C.c_int, C.c_int, _c_ip, C.c_int,
                                       C.POINTER(C.c_ulonglong)]),
    ("dci_b200_mdci_destroy", C.c_int, [_vp]),
    ("dci_b200_mdci_num_devices", C.c_int, [_vp]),
    ("dci_b200_mdci_shard", _vp, [_vp, C.c_int]),
    ("dci_b200_mdci_data_per_device", C.c_longlong, [_vp]),
    ("dci_b200_mdci_add", C.c_int, [_vp, _vp, C.c_longlong, C.c_int, C.c_int]),
    ("dci_b200_mdci_clear", C.c_int, [_vp]),
    ("dci_b200_mdci_query", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    ("dci_b200_mdci_query_host", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp]),
]

ERR_ARG, ERR_STATE, ERR_CUDA, ERR_UNSUPPORTED = 1, 2, 3, 4

_lib = None


class DCIError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


def lib():
    """Loads libdci_b200.so (built by dciknn_cuda_b200/build.py).  No fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "dciknn_cuda_b200: %s is missing; build it with `python -m dciknn_cuda_b200.build` "
                "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        handle = C.CDLL(LIB_PATH)
        for name, res, args in SYMBOLS:
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    """Maps a non-zero status to the exception class the reference's Python
    layer would raise for the same mistake (dciknn_cuda/core.py:53-71)."""
    if rc == 0:
        return
    msg = lib().dci_b200_last_error().decode("utf-8", "replace")
    if rc == ERR_ARG:
        raise ValueError(msg)
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise DCIError(rc, msg)
