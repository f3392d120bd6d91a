"""The backward entry point for callers that may not allocate: na2d_backward_static_scratch.

Some users of the library cannot call cudaMalloc at the point where they need the backward:
a plugin running inside a runtime whose memory arena already owns the whole GPU and offers no
workspace, or a training step that cannot afford the device-wide synchronisation cudaMalloc and
cudaFree bring.  For them the library keeps the backward's one scratch buffer (the row deltas the
dQ kernel passes to the dK/dV kernel) in a fixed array inside the library itself.  This file
checks, through the C ABI, that the variant gives what the ordinary entry point gives, twice in
a row (the array is shared between calls and keeps the previous call's contents), and that it
refuses problems larger than the array.  It is collected last so that a run stopping at the
first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

import e_natten_b200 as na
from e_natten_b200 import _lib
from e_natten_b200.functional import _DTYPES
from helpers import assert_close, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _both_backwards(shape, ks, dtype, seed):
    """dQ, dK, dV from na2d_backward (caller-provided delta) and from the static-scratch variant."""
    B, N, H, W, Cd = shape
    q, k, v, d_o = (t.to(DEV) for t in make_inputs(shape, dtype, seed, q_scale=Cd ** -0.5))
    o, lse = na.natten2d_forward(q, k, v, ks)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    geom = (B, N, H, W, Cd, ks, _DTYPES[dtype], None, _lib.PATH_AUTO, 0, st)

    ref = [torch.empty_like(q) for _ in range(3)]
    delta = torch.empty((B, N, H, W), dtype=torch.float32, device=DEV)
    _lib.check(_lib.lib.na2d_backward(_p(q), _p(k), _p(v), _p(o), _p(lse), _p(d_o), _p(ref[0]), _p(ref[1]),
                                      _p(ref[2]), _p(delta), *geom))
    got = [torch.full_like(q, float("nan")) for _ in range(3)]
    _lib.check(_lib.lib.na2d_backward_static_scratch(_p(q), _p(k), _p(v), _p(o), _p(lse), _p(d_o), _p(got[0]),
                                                     _p(got[1]), _p(got[2]), *geom))
    na.check_kernels(DEV)
    return got, ref


def test_static_scratch_backward_matches_ordinary_backward_twice_in_a_row():
    # call 1: bf16 on the tensor-core kernels; call 2: a smaller fp32 problem on the SIMT kernels,
    # which reuses the front of the array while the rest still holds call 1's deltas
    for shape, ks, dtype, seed in (((2, 2, 40, 48, 128), 5, torch.bfloat16, 11),
                                   ((1, 2, 16, 16, 32), 7, torch.float32, 12)):
        got, ref = _both_backwards(shape, ks, dtype, seed)
        for name, a, b in zip(("dq", "dk", "dv"), got, ref):
            assert_close(a, b.double(), dtype, f"{name} static-scratch vs ordinary, {shape} {dtype}")
            assert torch.equal(a, b), f"{name}: same kernels, same inputs, yet different bits"


def test_static_scratch_backward_refuses_what_does_not_fit():
    limit = 1 << 20
    B, N, H, W, Cd = 1, 1, 1032, 1024, 32                       # 1032*1024 > 2**20 row deltas
    assert B * N * H * W > limit
    one = torch.zeros(8, device=DEV)                             # never touched: the check comes first
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib.na2d_backward_static_scratch(*([_p(one)] * 9), B, N, H, W, Cd, 5, _lib.DTYPE_BF16, None,
                                               _lib.PATH_AUTO, 0, st)
    assert rc == _lib.ERR_TOO_LARGE
    msg = _lib.lib.na2d_last_cuda_error().decode()
    assert "1048576" in msg and str(B * N * H * W) in msg
    with pytest.raises(ValueError, match="size beyond"):
        _lib.check(rc)
    # exactly at the limit is accepted (B4 N4 256x256)
    assert 4 * 4 * 256 * 256 == limit
