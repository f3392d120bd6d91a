"""Host side of the fused 2D neighborhood attention: the drop-in for ``e_natten.natten2d``.

``natten2d(q, k, v, kernel_size=7)`` keeps the call signature, layout and autograd behaviour
of e_natten's fused entry point (e_natten/triton.py:487-550): tensors are
``(batch, heads, grid_rows, grid_cols, head_dim)``, the kernel size is odd, windows are
clamped at the borders, no softmax scale is applied, and the backward returns
``(dQ, dK, dV, None)``.  The arithmetic runs in libna2d.so (hand-written sm_100a CUDA behind a
C ABI); PyTorch only owns the memory and the stream.  There is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib

_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}
_PATHS = {"auto": _lib.PATH_AUTO, "simt": _lib.PATH_SIMT, "tensor": _lib.PATH_TENSOR}


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream(device: torch.device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_inputs(q, k, v, kernel_size, rows):
    if not (isinstance(q, torch.Tensor) and isinstance(k, torch.Tensor) and isinstance(v, torch.Tensor)):
        raise TypeError("q, k, v must be tensors")
    if q.dim() != 5:
        raise ValueError(f"q must be (B, heads, H, W, C); got {tuple(q.shape)}")
    if not q.is_cuda:
        raise ValueError("e_natten_b200 runs on CUDA tensors only (there is no CPU path)")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be on the same device")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must have the same dtype")
    if q.dtype not in _DTYPES:
        raise ValueError(f"dtype {q.dtype} not supported (float32, bfloat16, float16)")
    if k.shape != v.shape:
        raise ValueError("k and v must have the same shape")
    if not isinstance(kernel_size, int) or kernel_size <= 0 or kernel_size % 2 == 0:
        raise ValueError(f"kernel_size must be a positive odd integer; got {kernel_size!r}")
    if rows is None:
        if k.shape != q.shape:
            raise ValueError("q, k, v must have the same shape")
        H = q.shape[2]
    else:
        if k.shape[:2] != q.shape[:2] or k.shape[3:] != q.shape[3:]:
            raise ValueError("with a row view q and k may differ in the row dimension only")
        if q.shape[2] != rows.Hq or k.shape[2] != rows.Hkv:
            raise ValueError("row view does not match the tensors' row counts")
        H = rows.H_global
    if H < kernel_size or q.shape[3] < kernel_size:
        # e_natten/pytorch.py:7-11 produces a negative origin here and the reference reads
        # out of range; this library refuses instead.
        raise ValueError(f"grid {H}x{q.shape[3]} is smaller than kernel_size {kernel_size}")


def make_rows(q_row0: int, Hq: int, kv_row0: int, Hkv: int, H_global: int) -> _lib.Rows:
    """Row view for a caller that holds only a band of image rows (see include/na2d.h)."""
    return _lib.Rows(q_row0, Hq, kv_row0, Hkv, H_global)


def _geom_args(q, kernel_size, rows, path):
    B, N, H, W, Cd = q.shape
    return (B, N, H, W, Cd, kernel_size, _DTYPES[q.dtype], C.byref(rows) if rows is not None else None,
            _PATHS[path], q.device.index, _stream(q.device))


def forward_into(q, k, v, o, lse, kernel_size: int, rows=None, path: str = "auto") -> None:
    """Launch the forward into caller-owned ``o`` / ``lse`` (contiguous; nothing is allocated)."""
    _lib.check(_lib.lib.na2d_forward(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse),
                                     *_geom_args(q, kernel_size, rows, path)))


def backward_dq_into(q, k, v, o, lse, d_o, d_q, delta, kernel_size: int, rows=None, path: str = "auto") -> None:
    """Launch the query half of the backward: writes ``d_q`` (may be None) and ``delta``."""
    _lib.check(_lib.lib.na2d_backward_dq(_ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse), _ptr(d_o),
                                         _ptr(d_q), _ptr(delta), *_geom_args(q, kernel_size, rows, path)))


def backward_dkdv_into(q, k, v, lse, d_o, delta, d_k, d_v, kernel_size: int, rows=None, path: str = "auto") -> None:
    """Launch the key half of the backward: reads ``delta``, writes ``d_k`` and ``d_v``."""
    _lib.check(_lib.lib.na2d_backward_dkdv(_ptr(q), _ptr(k), _ptr(v), _ptr(lse), _ptr(d_o), _ptr(delta),
                                           _ptr(d_k), _ptr(d_v), *_geom_args(q, kernel_size, rows, path)))


def natten2d_forward(q, k, v, kernel_size: int, rows: Optional[_lib.Rows] = None,
                     path: str = "auto") -> Tuple[torch.Tensor, torch.Tensor]:
    """Raw forward: returns ``(o, lse)``; ``lse`` is fp32 ``(B, heads, H, W)``.  No autograd."""
    _check_inputs(q, k, v, kernel_size, rows)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, N, H, W, Cd = q.shape
    o = torch.empty_like(q)
    lse = torch.empty((B, N, H, W), dtype=torch.float32, device=q.device)
    if q.numel() == 0:
        return o, lse
    forward_into(q, k, v, o, lse, kernel_size, rows, path)
    return o, lse


def natten2d_backward(q, k, v, o, lse, d_o, kernel_size: int, rows: Optional[_lib.Rows] = None,
                      path: str = "auto", need_dq: bool = True, need_dkdv: bool = True):
    """Raw backward: returns ``(dQ, dK, dV)`` (``None`` for a half that was not asked for).

    With a row view dK / dV have the key band's shape and hold the partial sums over the local
    query band.
    """
    _check_inputs(q, k, v, kernel_size, rows)
    q, k, v, o, d_o = (t.contiguous() for t in (q, k, v, o, d_o))
    if d_o.shape != q.shape or d_o.dtype != q.dtype:
        raise ValueError("grad_output must match q in shape and dtype")
    B, N, H, W, Cd = q.shape
    d_q = torch.empty_like(q) if need_dq else None
    d_k = torch.empty_like(k) if need_dkdv else None
    d_v = torch.empty_like(v) if need_dkdv else None
    if q.numel() == 0 or not (need_dq or need_dkdv):
        return d_q, d_k, d_v
    delta = torch.empty((B, N, H, W), dtype=torch.float32, device=q.device)
    # the query half always runs: it produces delta = rowsum(dO * o) for the key half
    backward_dq_into(q, k, v, o, lse, d_o, d_q, delta, kernel_size, rows, path)
    if need_dkdv:
        backward_dkdv_into(q, k, v, lse, d_o, delta, d_k, d_v, kernel_size, rows, path)
    return d_q, d_k, d_v


class Natten2d(torch.autograd.Function):
    """Autograd wrapper with the reference's semantics (e_natten/triton.py:487-548); saves
    ``(q, k, v, o, lse)`` where the reference saves ``(Q, K, V, o)`` and recomputes the softmax."""

    @staticmethod
    def forward(ctx, q, k, v, kernel_size=7):
        o, lse = natten2d_forward(q, k, v, kernel_size)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.kernel_size = kernel_size
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, grad_output, _grad_lse):
        q, k, v, o, lse = ctx.saved_tensors
        need_dq = ctx.needs_input_grad[0]
        need_dkdv = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        d_q, d_k, d_v = natten2d_backward(q, k, v, o, lse, grad_output, ctx.kernel_size,
                                          need_dq=need_dq, need_dkdv=need_dkdv)
        return (d_q if ctx.needs_input_grad[0] else None,
                d_k if ctx.needs_input_grad[1] else None,
                d_v if ctx.needs_input_grad[2] else None, None)


def natten2d(q, k, v, kernel_size=7):
    """Fused 2D neighborhood attention, differentiable; drop-in for ``e_natten.natten2d``."""
    return Natten2d.apply(q, k, v, kernel_size)[0]


def natten2d_with_lse(q, k, v, kernel_size=7):
    """Like :func:`natten2d` but also returns the (non-differentiable) fp32 row log-sum-exp."""
    return Natten2d.apply(q, k, v, kernel_size)


# ---- index helpers with the reference's names (e_natten/pytorch.py:7-23) ------------------------
def get_window_start(i: int, seq_len: int, kernel_size: int) -> int:
    return _lib.lib.na2d_window_start(i, seq_len, kernel_size)


def get_backward_window_start(i: int, kernel_size: int) -> int:
    lo, hi = C.c_int(), C.c_int()
    _lib.check(_lib.lib.na2d_backward_window(i, max(i + 1, kernel_size), kernel_size, C.byref(lo), C.byref(hi)))
    return lo.value


def get_backward_window_end(i: int, seq_len: int, kernel_size: int) -> int:
    lo, hi = C.c_int(), C.c_int()
    _lib.check(_lib.lib.na2d_backward_window(i, seq_len, kernel_size, C.byref(lo), C.byref(hi)))
    return hi.value


def device_index_tables(seq_len: int, kernel_size: int, device="cuda:0"):
    """(ws, bws, bwe) int32 tensors computed on the device by the kernels' own index code."""
    dev = torch.device(device)
    ws, bws, bwe = (torch.empty(seq_len, dtype=torch.int32, device=dev) for _ in range(3))
    _lib.check(_lib.lib.na2d_dump_index(_ptr(ws), _ptr(bws), _ptr(bwe), seq_len, kernel_size,
                                        dev.index or 0, _stream(dev)))
    return ws, bws, bwe


def check_kernels(device="cuda:0") -> None:
    """Synchronise and raise if a kernel reported that a bounded wait ran out."""
    dev = torch.device(device)
    _lib.check(_lib.lib.na2d_check(dev.index or 0, _stream(dev)))


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(_lib.lib.na2d_launch_count())
