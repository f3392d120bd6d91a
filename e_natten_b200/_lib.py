"""ctypes binding of libna2d.so (the C ABI declared in include/na2d.h).

There is no fallback: if the shared library is missing or does not load, importing this
module raises, and every call that returns a non-zero status raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("NA2D_LIB", os.path.join(_PKG_DIR, "libna2d.so"))

DTYPE_F32, DTYPE_BF16, DTYPE_F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TENSOR = 0, 1, 2

ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WINDOW, ERR_CUDA = -1, -2, -3, -4
ERR_NO_DEVICE, ERR_TOO_LARGE, ERR_KERNEL_WAIT = -5, -6, -7


class Rows(C.Structure):
    """Mirror of ``na2d_rows``: which global image rows the query-side and key-side tensors hold."""
    _fields_ = [("q_row0", C.c_int), ("Hq", C.c_int), ("kv_row0", C.c_int), ("Hkv", C.c_int),
                ("H_global", C.c_int)]


class TensorDesc(C.Structure):
    """Mirror of ``na2d_tensor``: device pointer and element strides (batch, head, row, column);
    all strides zero means dense."""
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_n", C.c_int64),
                ("stride_h", C.c_int64), ("stride_w", C.c_int64)]


class Args(C.Structure):
    """Mirror of ``na2d_args``: everything one of the ``*_ex`` entry points needs."""
    _fields_ = [("struct_size", C.c_size_t), ("op", C.c_int),
                ("B", C.c_int), ("N", C.c_int), ("H", C.c_int), ("W", C.c_int), ("C", C.c_int),
                ("kernel_size", C.c_int), ("dtype", C.c_int), ("path", C.c_int), ("device", C.c_int),
                ("flags", C.c_int), ("scale", C.c_float), ("stream", C.c_void_p), ("rows", C.POINTER(Rows)),
                ("q", TensorDesc), ("k", TensorDesc), ("v", TensorDesc), ("o", TensorDesc),
                ("d_o", TensorDesc), ("d_q", TensorDesc), ("d_k", TensorDesc), ("d_v", TensorDesc),
                ("lse", C.c_void_p), ("delta", C.c_void_p)]


OP_2D, OP_1D = 0, 1
FLAG_DKDV_F32 = 1


def flag_sm_margin(n: int) -> int:
    """NA2D_FLAG_SM_MARGIN(n): the persistent kernels leave ``n`` SMs to a kernel running beside them."""
    return (int(n) & 0xFF) << 8
_DENSE = [C.c_int] * 7 + [C.POINTER(Rows), C.c_int, C.c_int, C.c_void_p]      # B..dtype, rows, path, device, stream
_PAIR = [C.c_int] * 7 + [C.c_int, C.c_void_p]                                  # B..dtype, device, stream

# name -> (restype, argtypes); every symbol include/na2d.h declares
SIGNATURES = {
    "na2d_version": (C.c_int, []),
    "na2d_strerror": (C.c_char_p, [C.c_int]),
    "na2d_last_cuda_error": (C.c_char_p, []),
    "na2d_window_start": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "na2d_backward_window": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "na2d_dump_index": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "na2d_forward": (C.c_int, [C.c_void_p] * 5 + _DENSE),
    "na2d_backward_dq": (C.c_int, [C.c_void_p] * 8 + _DENSE),
    "na2d_backward_dkdv": (C.c_int, [C.c_void_p] * 8 + _DENSE),
    "na2d_backward": (C.c_int, [C.c_void_p] * 10 + _DENSE),
    "na2d_backward_static_scratch": (C.c_int, [C.c_void_p] * 9 + _DENSE),
    "na2d_forward_ex": (C.c_int, [C.POINTER(Args)]),
    "na2d_backward_dq_ex": (C.c_int, [C.POINTER(Args)]),
    "na2d_backward_dkdv_ex": (C.c_int, [C.POINTER(Args)]),
    "na2d_backward_ex": (C.c_int, [C.POINTER(Args)]),
    "na1d_forward": (C.c_int, [C.c_void_p] * 5 + [C.c_int] * 6 + [C.c_int, C.c_void_p]),
    "na1d_backward": (C.c_int, [C.c_void_p] * 10 + [C.c_int] * 6 + [C.c_int, C.c_void_p]),
    "na2d_qk_forward": (C.c_int, [C.c_void_p] * 3 + _PAIR),
    "na2d_qk_backward": (C.c_int, [C.c_void_p] * 5 + _PAIR),
    "na2d_av_forward": (C.c_int, [C.c_void_p] * 3 + _PAIR),
    "na2d_av_backward": (C.c_int, [C.c_void_p] * 5 + _PAIR),
    "na2d_check": (C.c_int, [C.c_int, C.c_void_p]),
    "na2d_poll": (C.c_int, [C.c_int, C.c_void_p]),
    "na2d_selftest_wait_timeout": (C.c_int, [C.c_int, C.c_void_p, C.c_uint]),
    "na2d_launch_count": (C.c_longlong, []),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. Run "
            "`python e_natten_b200/build.py` (needs nvcc); there is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} is stale (no symbol {name}); rebuild it with "
                              "`python e_natten_b200/build.py --force`") from exc
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class Na2dError(RuntimeError):
    def __init__(self, status: int):
        self.status = status
        msg = lib.na2d_strerror(status).decode()
        if status == ERR_CUDA:
            msg += " -- " + lib.na2d_last_cuda_error().decode()
        super().__init__(f"libna2d status {status}: {msg}")


def check(status: int) -> None:
    """Raise for a non-zero status: ValueError for argument problems, RuntimeError otherwise."""
    if status == 0:
        return
    err = Na2dError(status)
    if status in (ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WINDOW, ERR_TOO_LARGE):
        raise ValueError(str(err))
    raise err
