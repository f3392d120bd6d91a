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


def test_static_scratch_backward_allocates_nothing_once_warm_and_takes_a_row_view():
    """After one warm-up call on the device (which makes the runtime load the library's device code,
    the built-in array with it) a call changes neither the device's free memory nor what the
    framework's allocator holds.  Run at the largest shape that fits (B4 N4 256x256) and, a second
    time, on a row band of it through na2d_rows."""
    B, N, H, W, Cd, ks, dtype = 4, 4, 256, 256, 32, 5, torch.bfloat16
    assert B * N * H * W == 1 << 20
    q, k, v, d_o = (torch.randn((B, N, H, W, Cd), device=DEV).mul(0.5).to(dtype) for _ in range(4))
    o, lse = na.natten2d_forward(q, k, v, ks)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = [torch.empty_like(q) for _ in range(3)]

    def call(rows, qq, kk, vv, oo, ll, gg, dq, dk, dv):
        b, n, h, w, c = qq.shape
        return _lib.lib.na2d_backward_static_scratch(_p(qq), _p(kk), _p(vv), _p(oo), _p(ll), _p(gg), _p(dq), _p(dk), _p(dv),
                                                     b, n, h, w, c, ks, _DTYPES[dtype], rows, _lib.PATH_AUTO, 0, st)

    _lib.check(call(None, q, k, v, o, lse, d_o, *outs))              # warm-up: first use of the array on this device
    torch.cuda.synchronize()
    free0, held0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    _lib.check(call(None, q, k, v, o, lse, d_o, *outs))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == held0
    na.check_kernels(DEV)
    ref = na.natten2d_backward(q, k, v, o, lse, d_o, ks)
    for name, a, b in zip(("dq", "dk", "dv"), outs, ref):
        assert torch.equal(a, b), f"{name} at the largest shape that fits"
    # a row band of the same image: query rows [96, 160), the key rows their windows reach
    a0, a1 = 96, 160
    kv0 = na.get_window_start(a0, H, ks)
    kv1 = na.get_window_start(a1 - 1, H, ks) + ks
    rows = na.make_rows(a0, a1 - a0, kv0, kv1 - kv0, H)
    qb, ob, lb, gb = (t[:, :, a0:a1].contiguous() for t in (q, o, lse, d_o))
    kb, vb = k[:, :, kv0:kv1].contiguous(), v[:, :, kv0:kv1].contiguous()
    got = [torch.empty_like(qb), torch.empty_like(kb), torch.empty_like(vb)]
    _lib.check(call(C.byref(rows), qb, kb, vb, ob, lb, gb, *got))
    na.check_kernels(DEV)
    want = na.natten2d_backward(qb, kb, vb, ob, lb, gb, ks, rows=rows)
    for name, a, b in zip(("dq", "dk", "dv"), got, want):
        assert torch.equal(a, b), f"{name} under a row view"


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
