"""Host side of the fused neighborhood attention: the drop-in for ``e_natten.natten2d`` /
``e_natten.natten1d``.

``natten2d(q, k, v, kernel_size=7)`` keeps the call signature, layout and autograd behaviour
of e_natten's fused entry point (e_natten/triton.py:487-550): tensors are
``(batch, heads, grid_rows, grid_cols, head_dim)``, the kernel size is odd, windows are
clamped at the borders, and the backward returns ``(dQ, dK, dV, None)``.  ``natten1d`` is the
same for ``(batch, heads, tokens, head_dim)`` (e_natten/triton.py:425-485).  The arithmetic runs
in libna2d.so (hand-written sm_100a CUDA behind a C ABI); PyTorch only owns the memory and the
stream.  There is no CPU path.

Two things the reference leaves to its caller are arguments here: a softmax ``scale`` (the
reference applies none, e_natten/triton.py:280, so callers multiply q beforehand) and strided
inputs (the reference asserts equal strides, e_natten/triton.py:233-234): views of a packed
``(B, H, W, 3, heads, C)`` qkv projection go to the kernels as they are, without copies.
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


# ---- layouts ---------------------------------------------------------------------------------------
def _kernel_ready(t: torch.Tensor) -> bool:
    """True if the kernels can read ``t`` in place: channels contiguous and, for the 16-bit
    tensor-core path (TMA tensor maps), a 16-byte aligned base and strides that are multiples
    of 16 bytes.  fp32 tensors (SIMT kernels) only need contiguous channels."""
    if t.numel() == 0:
        return True
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        return False
    if any(s < 0 for s in t.stride()):
        return False
    if t.element_size() == 2:
        if t.data_ptr() % 16:
            return False
        for size, stride in zip(t.shape[:-1], t.stride()[:-1]):
            if size > 1 and (stride % 8 or stride == 0):
                return False
    else:
        for size, stride in zip(t.shape[:-1], t.stride()[:-1]):
            if size > 1 and stride == 0:
                return False
    return True


def as_kernel_input(t: torch.Tensor) -> torch.Tensor:
    """``t`` itself when the kernels can read it in place (any batch / head / row / column strides
    with contiguous channels), else a dense copy."""
    return t if _kernel_ready(t) else t.contiguous()


def _desc(t: Optional[torch.Tensor]) -> _lib.TensorDesc:
    if t is None:
        return _lib.TensorDesc(None, 0, 0, 0, 0)
    if t.dim() == 5:
        sb, sn, sh, sw, _ = t.stride()
    else:                                     # (B, N, T, C): the 1D operator, a one-row image
        sb, sn, sw, _ = t.stride()
        sh = 0
    # a dimension of extent 1 may report any stride; the library ignores it, but all-zero means dense
    return _lib.TensorDesc(t.data_ptr(), max(sb, 1), max(sn, 1), max(sh, 1) if t.dim() == 5 else 0, max(sw, 1))


def _args(like, kernel_size: int, rows, path: str, scale: float, **tensors) -> _lib.Args:
    """na2d_args for a problem shaped like the query tensor ``like``; ``tensors`` are the operands by
    their field names."""
    a = _lib.Args()
    a.struct_size = C.sizeof(_lib.Args)
    if like.dim() == 5:
        a.op = _lib.OP_2D
        a.B, a.N, a.H, a.W, a.C = like.shape
    else:
        a.op = _lib.OP_1D
        a.B, a.N, a.W, a.C = like.shape
        a.H = 1
    a.kernel_size = kernel_size
    a.dtype = _DTYPES[like.dtype]
    a.path = _PATHS[path]
    a.device = like.device.index or 0
    a.scale = float(scale)
    a.stream = torch.cuda.current_stream(like.device).cuda_stream if like.is_cuda else None
    a.rows = C.pointer(rows) if rows is not None else None
    for name, t in tensors.items():
        if name in ("lse", "delta"):
            setattr(a, name, 0 if t is None else t.data_ptr())
        else:
            setattr(a, name, _desc(t))
    return a


# ---- raw launches into caller-owned buffers ------------------------------------------------------------
def forward_into(q, k, v, o, lse, kernel_size: int, rows=None, path: str = "auto", scale: float = 1.0,
                 sm_margin: int = 0) -> None:
    """Launch the forward into caller-owned ``o`` / ``lse``; nothing is allocated.  ``sm_margin``
    SMs are left free for a kernel that should run beside this one (a halo exchange)."""
    a = _args(q, kernel_size, rows, path, scale, q=q, k=k, v=v, o=o, lse=lse)
    a.flags |= _lib.flag_sm_margin(sm_margin)
    _lib.check(_lib.lib.na2d_forward_ex(C.byref(a)))


def backward_dq_into(q, k, v, o, lse, d_o, d_q, delta, kernel_size: int, rows=None, path: str = "auto",
                     scale: float = 1.0) -> None:
    """Launch the query half of the backward: writes ``d_q`` (may be None) and ``delta``.  ``o`` may be
    None; with it the kernels of the larger windows take the faster one-walk form."""
    a = _args(q, kernel_size, rows, path, scale, q=q, k=k, v=v, o=o, lse=lse, d_o=d_o, d_q=d_q, delta=delta)
    _lib.check(_lib.lib.na2d_backward_dq_ex(C.byref(a)))


def backward_dkdv_into(q, k, v, lse, d_o, delta, d_k, d_v, kernel_size: int, rows=None, path: str = "auto",
                       scale: float = 1.0, sm_margin: int = 0) -> None:
    """Launch the key half of the backward: reads ``delta``, writes ``d_k`` and ``d_v``, which have
    the inputs' dtype or, for 16-bit inputs, may both be fp32 (partial sums of a row band)."""
    a = _args(q, kernel_size, rows, path, scale, q=q, k=k, v=v, lse=lse, d_o=d_o, delta=delta, d_k=d_k, d_v=d_v)
    if d_k.dtype != q.dtype:
        if d_k.dtype != torch.float32 or d_v.dtype != torch.float32:
            raise ValueError("d_k and d_v must have the inputs' dtype or both be float32")
        a.flags |= _lib.FLAG_DKDV_F32
    a.flags |= _lib.flag_sm_margin(sm_margin)
    _lib.check(_lib.lib.na2d_backward_dkdv_ex(C.byref(a)))


# ---- 2D operator ----------------------------------------------------------------------------------------
def natten2d_forward(q, k, v, kernel_size: int, rows: Optional[_lib.Rows] = None, path: str = "auto",
                     scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Raw forward: returns ``(o, lse)``; ``lse`` is fp32 ``(B, heads, H, W)``.  No autograd."""
    _check_inputs(q, k, v, kernel_size, rows)
    q, k, v = as_kernel_input(q), as_kernel_input(k), as_kernel_input(v)
    B, N, H, W, Cd = q.shape
    o = torch.empty((B, N, H, W, Cd), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, N, H, W), dtype=torch.float32, device=q.device)
    if q.numel() != 0:
        forward_into(q, k, v, o, lse, kernel_size, rows, path, scale)
    return o, lse


def natten2d_backward(q, k, v, o, lse, d_o, kernel_size: int, rows: Optional[_lib.Rows] = None,
                      path: str = "auto", need_dq: bool = True, need_dkdv: bool = True, scale: float = 1.0,
                      dkdv_dtype: Optional[torch.dtype] = None):
    """Raw backward: returns ``(dQ, dK, dV)`` (``None`` for a half that was not asked for).

    With a row view dK / dV have the key band's shape and hold the partial sums over the local
    query band; ``dkdv_dtype=torch.float32`` keeps those partial sums in fp32.
    """
    _check_inputs(q, k, v, kernel_size, rows)
    q, k, v, d_o = (as_kernel_input(t) for t in (q, k, v, d_o))
    if d_o.shape != q.shape or d_o.dtype != q.dtype:
        raise ValueError("grad_output must match q in shape and dtype")
    if o is not None:
        o = as_kernel_input(o)
    B, N, H, W, Cd = q.shape
    d_q = torch.empty(q.shape, dtype=q.dtype, device=q.device) if need_dq else None
    d_k = torch.empty(k.shape, dtype=dkdv_dtype or k.dtype, device=q.device) if need_dkdv else None
    d_v = torch.empty(v.shape, dtype=dkdv_dtype or v.dtype, device=q.device) if need_dkdv else None
    if q.numel() == 0 or not (need_dq or need_dkdv):
        return d_q, d_k, d_v
    delta = torch.empty((B, N, H, W), dtype=torch.float32, device=q.device)
    # the query half always runs: it produces delta = rowsum(dO * o) for the key half
    backward_dq_into(q, k, v, o, lse, d_o, d_q, delta, kernel_size, rows, path, scale)
    if need_dkdv:
        backward_dkdv_into(q, k, v, lse, d_o, delta, d_k, d_v, kernel_size, rows, path, scale)
    return d_q, d_k, d_v


def poll_kernels(device) -> None:
    """Raise if a kernel of an earlier call on ``device`` reported that a bounded wait ran out.
    Never waits for the GPU: it looks at the answer to the question the previous poll asked and
    asks again (``na2d_poll``), so an error surfaces one call late."""
    dev = torch.device(device)
    _lib.check(_lib.lib.na2d_poll(dev.index or 0, _stream(dev)))


class Natten2d(torch.autograd.Function):
    """Autograd wrapper with the reference's semantics (e_natten/triton.py:487-548); saves
    ``(q, k, v, o, lse)`` where the reference saves ``(Q, K, V, o)`` and recomputes the softmax."""

    @staticmethod
    def forward(ctx, q, k, v, kernel_size=7, scale=None):
        scale = 1.0 if scale is None else float(scale)
        o, lse = natten2d_forward(q, k, v, kernel_size, scale=scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.kernel_size, ctx.scale = kernel_size, scale
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, grad_output, _grad_lse):
        q, k, v, o, lse = ctx.saved_tensors
        poll_kernels(q.device)            # a wait that gave up in an earlier kernel surfaces here, without a sync
        need_dq = ctx.needs_input_grad[0]
        need_dkdv = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        d_q, d_k, d_v = natten2d_backward(q, k, v, o, lse, grad_output, ctx.kernel_size,
                                          need_dq=need_dq, need_dkdv=need_dkdv, scale=ctx.scale)
        return (d_q if ctx.needs_input_grad[0] else None,
                d_k if ctx.needs_input_grad[1] else None,
                d_v if ctx.needs_input_grad[2] else None, None, None)


def natten2d(q, k, v, kernel_size=7, scale=None):
    """Fused 2D neighborhood attention, differentiable; drop-in for ``e_natten.natten2d``.
    ``scale`` (default: none, as in the reference) multiplies the logits inside the kernels."""
    return Natten2d.apply(q, k, v, kernel_size, scale)[0]


def natten2d_with_lse(q, k, v, kernel_size=7, scale=None):
    """Like :func:`natten2d` but also returns the (non-differentiable) fp32 row log-sum-exp."""
    return Natten2d.apply(q, k, v, kernel_size, scale)


# ---- 1D operator ------------------------------------------------------------------------------------------
def _check_inputs_1d(q, k, v, kernel_size):
    if not (isinstance(q, torch.Tensor) and isinstance(k, torch.Tensor) and isinstance(v, torch.Tensor)):
        raise TypeError("q, k, v must be tensors")
    if q.dim() != 4:
        raise ValueError(f"q must be (B, heads, T, C); got {tuple(q.shape)}")
    if not q.is_cuda:
        raise ValueError("e_natten_b200 runs on CUDA tensors only (there is no CPU path)")
    if k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must have the same shape")
    if k.dtype != q.dtype or v.dtype != q.dtype or q.dtype not in _DTYPES:
        raise ValueError("q, k, v must share one dtype of float32, bfloat16, float16")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be on the same device")
    if not isinstance(kernel_size, int) or kernel_size <= 0 or kernel_size % 2 == 0:
        raise ValueError(f"kernel_size must be a positive odd integer; got {kernel_size!r}")
    if q.shape[2] < kernel_size:
        raise ValueError(f"sequence of {q.shape[2]} tokens is shorter than kernel_size {kernel_size}")


def natten1d_forward(q, k, v, kernel_size: int, scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Raw 1D forward on ``(B, heads, T, C)``: returns ``(o, lse)``, lse fp32 ``(B, heads, T)``."""
    _check_inputs_1d(q, k, v, kernel_size)
    q, k, v = as_kernel_input(q), as_kernel_input(k), as_kernel_input(v)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    if q.numel() != 0:
        a = _args(q, kernel_size, None, "auto", scale, q=q, k=k, v=v, o=o, lse=lse)
        _lib.check(_lib.lib.na2d_forward_ex(C.byref(a)))
    return o, lse


def natten1d_backward(q, k, v, o, lse, d_o, kernel_size: int, need_dq: bool = True, need_dkdv: bool = True,
                      scale: float = 1.0):
    """Raw 1D backward: ``(dQ, dK, dV)``."""
    _check_inputs_1d(q, k, v, kernel_size)
    q, k, v, d_o = (as_kernel_input(t) for t in (q, k, v, d_o))
    if d_o.shape != q.shape or d_o.dtype != q.dtype:
        raise ValueError("grad_output must match q in shape and dtype")
    d_q = torch.empty(q.shape, dtype=q.dtype, device=q.device) if need_dq else None
    d_k = torch.empty(q.shape, dtype=q.dtype, device=q.device) if need_dkdv else None
    d_v = torch.empty(q.shape, dtype=q.dtype, device=q.device) if need_dkdv else None
    if q.numel() == 0 or not (need_dq or need_dkdv):
        return d_q, d_k, d_v
    delta = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    a = _args(q, kernel_size, None, "auto", scale, q=q, k=k, v=v, lse=lse, d_o=d_o, d_q=d_q, d_k=d_k, d_v=d_v,
              delta=delta)
    _lib.check(_lib.lib.na2d_backward_ex(C.byref(a)))
    return d_q, d_k, d_v


class Natten1d(torch.autograd.Function):
    """Autograd wrapper of the 1D operator with the reference's semantics
    (e_natten/triton.py:425-485): ``forward(ctx, q, k, v, kernel_size=7)``, backward returns
    ``(dQ, dK, dV, None)``."""

    @staticmethod
    def forward(ctx, q, k, v, kernel_size=7, scale=None):
        scale = 1.0 if scale is None else float(scale)
        o, lse = natten1d_forward(q, k, v, kernel_size, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.kernel_size, ctx.scale = kernel_size, scale
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, o, lse = ctx.saved_tensors
        need_dq = ctx.needs_input_grad[0]
        need_dkdv = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        d_q, d_k, d_v = natten1d_backward(q, k, v, o, lse, grad_output, ctx.kernel_size, need_dq, need_dkdv,
                                          ctx.scale)
        return (d_q if ctx.needs_input_grad[0] else None,
                d_k if ctx.needs_input_grad[1] else None,
                d_v if ctx.needs_input_grad[2] else None, None, None)


def natten1d(q, k, v, kernel_size=7, scale=None):
    """Fused 1D neighborhood attention, differentiable; drop-in for ``e_natten.natten1d``."""
    return Natten1d.apply(q, k, v, kernel_size, scale)


# ---- the unfused pair (scores, apply) with the call shape of natten.functional --------------------------------
def _pair_args(t, kernel_size):
    B, N, H, W, Cd = t.shape
    return (B, N, H, W, Cd, kernel_size, _DTYPES[t.dtype], t.device.index, _stream(t.device))


def _check_pair(x, y, kernel_size, dilation):
    if dilation != 1:
        raise ValueError("only dilation 1 is built (the reference uses nothing else: test.py:17-21)")
    if x.dim() != 5 or y.dim() != 5 or not x.is_cuda or x.dtype not in _DTYPES or y.dtype != x.dtype:
        raise ValueError("expected two 5-D CUDA tensors of one supported dtype")
    if not isinstance(kernel_size, int) or kernel_size <= 0 or kernel_size % 2 == 0:
        raise ValueError(f"kernel_size must be a positive odd integer; got {kernel_size!r}")


class _Natten2dQK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, kernel_size, dilation):
        _check_pair(q, k, kernel_size, dilation)
        q, k = q.contiguous(), k.contiguous()
        B, N, H, W, _ = q.shape
        attn = torch.empty((B, N, H, W, kernel_size * kernel_size), dtype=q.dtype, device=q.device)
        _lib.check(_lib.lib.na2d_qk_forward(_ptr(q), _ptr(k), _ptr(attn), *_pair_args(q, kernel_size)))
        ctx.save_for_backward(q, k)
        ctx.kernel_size = kernel_size
        return attn

    @staticmethod
    def backward(ctx, d_attn):
        q, k = ctx.saved_tensors
        d_attn = d_attn.contiguous()
        d_q, d_k = torch.empty_like(q), torch.empty_like(k)
        _lib.check(_lib.lib.na2d_qk_backward(_ptr(q), _ptr(k), _ptr(d_attn), _ptr(d_q), _ptr(d_k),
                                             *_pair_args(q, ctx.kernel_size)))
        return d_q, d_k, None, None


class _Natten2dAV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn, v, kernel_size, dilation):
        _check_pair(attn, v, kernel_size, dilation)
        attn, v = attn.contiguous(), v.contiguous()
        if attn.shape[:4] != v.shape[:4] or attn.shape[4] != kernel_size * kernel_size:
            raise ValueError("attn must be (B, heads, H, W, kernel_size**2) for v of (B, heads, H, W, C)")
        out = torch.empty_like(v)
        _lib.check(_lib.lib.na2d_av_forward(_ptr(attn), _ptr(v), _ptr(out), *_pair_args(v, kernel_size)))
        ctx.save_for_backward(attn, v)
        ctx.kernel_size = kernel_size
        return out

    @staticmethod
    def backward(ctx, d_out):
        attn, v = ctx.saved_tensors
        d_out = d_out.contiguous()
        d_attn, d_v = torch.empty_like(attn), torch.empty_like(v)
        _lib.check(_lib.lib.na2d_av_backward(_ptr(attn), _ptr(v), _ptr(d_out), _ptr(d_attn), _ptr(d_v),
                                             *_pair_args(v, ctx.kernel_size)))
        return d_attn, d_v, None, None


def natten2dqk(query, key, kernel_size, dilation=1):
    """Neighborhood scores ``(B, heads, H, W, kernel_size**2)``: the first step of the unfused
    pair the reference's test and benchmark compare with (test.py:17, bench.py:23)."""
    return _Natten2dQK.apply(query, key, kernel_size, dilation)


def natten2dav(attn, value, kernel_size, dilation=1):
    """Applies neighborhood weights to the values: the second step of the unfused pair
    (test.py:21, bench.py:23)."""
    return _Natten2dAV.apply(attn, value, kernel_size, dilation)


def natten2d_unfused(q, k, v, kernel_size=7):
    """``natten2dav(softmax(natten2dqk(q, k)), v)``: the baseline of the reference's benchmark."""
    return natten2dav(torch.softmax(natten2dqk(q, k, kernel_size, 1), dim=-1), v, kernel_size, 1)


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
