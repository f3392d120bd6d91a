"""CPU tests of the C ABI: the library loads, exports what include/na2d.h declares, its host-side
index functions are bit-exact with the reference's, and bad arguments are refused before any CUDA
call.  No compute runs here."""
import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

import e_natten_b200 as na
from e_natten_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "na2d.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(na2d_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_functions()
    assert "na2d_forward" in names and "na2d_backward" in names and len(names) >= 10
    raw = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/na2d.h but not exported"
    assert sorted(_lib.SIGNATURES) == names               # the binding covers exactly the header


def test_version_and_strerror():
    assert _lib.lib.na2d_version() >= 100
    for code in range(0, -8, -1):
        assert len(_lib.lib.na2d_strerror(code)) > 0


@pytest.mark.parametrize("ks", list(range(3, 16, 2)))
def test_host_index_functions_bit_exact(golden, ks):
    for L in list(range(ks, 81)) + [192, 256, 1024]:
        ws = np.array([na.get_window_start(i, L, ks) for i in range(L)], dtype=np.int32)
        assert np.array_equal(ws, golden[f"idx/ws/{ks}/{L}"])
        if L <= 40 or L == 1024:
            bs = np.array([na.get_backward_window_start(i, ks) for i in range(L)], dtype=np.int32)
            be = np.array([na.get_backward_window_end(i, L, ks) for i in range(L)], dtype=np.int32)
            assert np.array_equal(bs, golden[f"idx/bws/{ks}/{L}"])
            assert np.array_equal(be, golden[f"idx/bwe/{ks}/{L}"])


def _fwd(ptrs=(1, 1, 1, 1, 1), B=1, N=1, H=8, W=8, Cd=32, ks=5, dtype=0, rows=None, path=0):
    p = [C.c_void_p(x) for x in ptrs]
    return _lib.lib.na2d_forward(*p, B, N, H, W, Cd, ks, dtype, rows, path, 0, None)


def test_forward_refuses_bad_arguments_without_touching_cuda():
    # (non-null dummy pointers are never dereferenced: validation comes first)
    assert _fwd(ptrs=(0, 1, 1, 1, 1)) == _lib.ERR_BAD_ARG
    assert _fwd(ks=4) == _lib.ERR_BAD_ARG
    assert _fwd(ks=-1) == _lib.ERR_BAD_ARG
    assert _fwd(B=0) == _lib.ERR_BAD_ARG
    assert _fwd(dtype=7) == _lib.ERR_UNSUPPORTED
    assert _fwd(H=4, ks=5) == _lib.ERR_WINDOW
    assert _fwd(W=3, ks=5) == _lib.ERR_WINDOW
    assert _fwd(Cd=512, path=_lib.PATH_SIMT) == _lib.ERR_UNSUPPORTED
    assert _fwd(dtype=0, path=_lib.PATH_TENSOR) == _lib.ERR_UNSUPPORTED      # fp32 has no tensor path
    assert _fwd(path=9) == _lib.ERR_BAD_ARG
    # row views: the key band must cover the query band's windows
    ok = _lib.Rows(8, 8, 6, 12, 32)
    assert _fwd(rows=C.byref(_lib.Rows(8, 8, 8, 8, 32))) == _lib.ERR_WINDOW
    assert _fwd(rows=C.byref(_lib.Rows(8, 8, 6, 9, 32))) == _lib.ERR_WINDOW
    assert _fwd(rows=C.byref(_lib.Rows(30, 8, 20, 12, 32))) == _lib.ERR_BAD_ARG
    assert _fwd(rows=C.byref(ok)) in (_lib.ERR_CUDA, _lib.ERR_NO_DEVICE)     # past validation: needs a GPU


def test_python_wrapper_refuses_cpu_tensors_and_bad_shapes():
    q = torch.zeros(1, 1, 8, 8, 32)
    with pytest.raises(ValueError, match="CUDA"):
        na.natten2d(q, q, q, 5)
    with pytest.raises(ValueError):
        na.natten2d(torch.zeros(1, 8, 8, 32), q, q, 5)
    with pytest.raises(TypeError):
        na.natten2d(None, q, q, 5)


def test_check_maps_status_to_exceptions():
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_WINDOW)
    with pytest.raises(RuntimeError):
        _lib.check(_lib.ERR_KERNEL_WAIT)
    _lib.check(0)
