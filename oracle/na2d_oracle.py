"""CPU oracle for fused 2D neighborhood attention.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the algorithm of e_natten's fused 2D
neighborhood attention so that the CUDA kernels can be checked against it.  It is
imported only by the test-suite, by the smoke check and by the benchmark's
CPU-baseline / reference arm; the product package never imports it.

Parity status: PINNED.  The restatement is checked against the reference's own
code (e_natten/pytorch.py run on CPU and e_natten/triton.py run under the Triton
interpreter) through the fixtures in tests/golden/, which
tests/golden/make_golden.py generates by importing the reference.

What follows which reference lines (paths inside the e_natten project):

* window_start            <- e_natten/pytorch.py:7-11  (get_window_start), the
                             device twin is e_natten/triton.py:7-12
* backward_window_start   <- e_natten/pytorch.py:13-17
* backward_window_end     <- e_natten/pytorch.py:19-23
* natten2d_pixel          <- e_natten/pytorch.py:192-202 / e_natten/triton.py:242-291
                             (one softmax(q.K_window) @ V_window per pixel; gradients
                             by autograd, which is what e_natten/triton.py:383-423
                             computes with an explicit Jacobian)
* natten2d_fwd / _bwd     <- the same math, vectorised over the k*k window offsets,
                             backward in the flash form dS = P*(dP - rowsum(dO*O)),
                             algebraically equal to diag(P) - P P^T applied to dP
                             (e_natten/pytorch.py:33-43, 250-257, 277-288)

* natten1d_pixel / _fwd / _bwd <- the 1D operator: e_natten/pytorch.py:46-156 (loop
                             restatement), e_natten/triton.py:65-222 (kernels); same math on
                             one axis, (B, N, T, C)
* natten2d_qk / natten2d_av <- the unfused pair the reference's test and benchmark compare
                             with (test.py:17-21, bench.py:23, 52-54): window scores and their
                             application, window member j at row j // ks, column j % ks

Layout everywhere: (B, N, H, W, C) = batch, heads, grid rows, grid cols, head dim
(e_natten/triton.py:500).  The reference applies no softmax scale (e_natten/triton.py:280);
``scale`` (default 1) multiplies the logits, as a caller-side ``q * scale`` would.
"""
from __future__ import annotations

import torch

__all__ = [
    "window_start", "backward_window_start", "backward_window_end",
    "window_start_table", "natten2d_pixel", "natten2d_fwd", "natten2d_bwd",
    "natten2d_fwd_bwd", "round_inputs",
    "natten1d_pixel", "natten1d_fwd", "natten1d_bwd", "natten2d_qk", "natten2d_av",
]


# --------------------------------------------------------------------------- index math
def window_start(i: int, seq_len: int, kernel_size: int) -> int:
    """Clamped window origin of pixel ``i`` (e_natten/pytorch.py:7-11)."""
    start = max(i - kernel_size // 2, 0)
    if i + kernel_size // 2 >= seq_len:
        start += seq_len - i - kernel_size // 2 - 1
    return start


def backward_window_start(i: int, kernel_size: int) -> int:
    """First query index whose window holds key ``i`` (e_natten/pytorch.py:13-17)."""
    return 0 if i < kernel_size else i - kernel_size // 2


def backward_window_end(i: int, seq_len: int, kernel_size: int) -> int:
    """One past the last query index whose window holds key ``i``
    (e_natten/pytorch.py:19-23)."""
    return seq_len if i >= seq_len - kernel_size else i + kernel_size // 2 + 1


def window_start_table(seq_len: int, kernel_size: int) -> torch.Tensor:
    """int64 vector of window_start(i) for i in [0, seq_len)."""
    return torch.tensor([window_start(i, seq_len, kernel_size) for i in range(seq_len)],
                        dtype=torch.int64)


# --------------------------------------------------------------------------- per pixel
def natten2d_pixel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel_size: int) -> torch.Tensor:
    """Differentiable per-pixel loop; the smallest possible statement of the op.

    For every pixel the k*k window at origin (ws(x,H), ws(y,W)) is sliced out of K
    and V and one softmax attention row is computed.  Only for small grids.
    """
    B, N, H, W, C = q.shape
    rows = []
    for x in range(H):
        ox = window_start(x, H, kernel_size)
        cols = []
        for y in range(W):
            oy = window_start(y, W, kernel_size)
            kw = k[:, :, ox:ox + kernel_size, oy:oy + kernel_size, :].reshape(B, N, kernel_size ** 2, C)
            vw = v[:, :, ox:ox + kernel_size, oy:oy + kernel_size, :].reshape(B, N, kernel_size ** 2, C)
            s = torch.matmul(q[:, :, x, y, :].unsqueeze(2), kw.transpose(-1, -2))
            p = torch.softmax(s, dim=-1)
            cols.append(torch.matmul(p, vw))          # (B, N, 1, C)
        rows.append(torch.cat(cols, dim=2))           # (B, N, W, C)
    return torch.stack(rows, dim=2)                   # (B, N, H, W, C)


# --------------------------------------------------------------------------- vectorised
def _shifted(t: torch.Tensor, wsx: torch.Tensor, wsy: torch.Tensor, u: int, w: int) -> torch.Tensor:
    """t[..., ws(x)+u, ws(y)+w, :] for every (x, y): the (u, w)-th window member."""
    return t.index_select(2, wsx + u).index_select(3, wsy + w)


def _row_origins(Hq: int, kernel_size: int, rows):
    """Window origins of the query rows as indices into the key-side tensor.

    ``rows`` = (q_row0, kv_row0, H_global) describes a band of a taller image: the query-side
    tensors hold global rows [q_row0, q_row0+Hq), the key-side tensors start at global row
    kv_row0, and clamping is against H_global.  None means the whole image.
    """
    if rows is None:
        return window_start_table(Hq, kernel_size)
    q_row0, kv_row0, h_global = rows
    return torch.tensor([window_start(q_row0 + x, h_global, kernel_size) - kv_row0 for x in range(Hq)],
                        dtype=torch.int64)


def natten2d_fwd(q, k, v, kernel_size: int, acc_dtype=torch.float64, rows=None, scale: float = 1.0):
    """Forward.  Returns (o, lse) in ``acc_dtype``; lse = max + log(sum exp), natural log.

    Loops over the k*k window offsets; each step is one full-tensor gather + dot.
    """
    B, N, H, W, C = q.shape
    ks = kernel_size
    q, k, v = q.to(acc_dtype) * scale, k.to(acc_dtype), v.to(acc_dtype)
    wsx, wsy = _row_origins(H, ks, rows), window_start_table(W, ks)
    s = torch.empty(ks * ks, B, N, H, W, dtype=acc_dtype)
    for u in range(ks):
        for w in range(ks):
            s[u * ks + w] = (q * _shifted(k, wsx, wsy, u, w)).sum(-1)
    m = s.max(dim=0).values
    e = torch.exp(s - m)
    l = e.sum(0)
    p = e / l
    o = torch.zeros_like(q)
    for u in range(ks):
        for w in range(ks):
            o += p[u * ks + w].unsqueeze(-1) * _shifted(v, wsx, wsy, u, w)
    return o, m + torch.log(l)


def natten2d_bwd(q, k, v, d_o, kernel_size: int, acc_dtype=torch.float64, rows=None, o=None, scale: float = 1.0):
    """Backward in flash form.  Returns (dq, dk, dv) in ``acc_dtype``.

    p = exp(s - lse), delta = dO.O, dS = p*(dO.V - delta), dQ = sum dS*K,
    dK[key] += dS*q and dV[key] += p*dO summed over every query whose window holds
    the key (scatter-add through the same window origins, so the inverse
    neighbourhood of e_natten/pytorch.py:261-273 is implied, not re-derived).
    With ``rows`` (see _row_origins) dk / dv have the key band's shape and hold the partial
    sums over the local query band.

    ``o`` is the forward output as the backward receives it.  The fused entry point saves o in
    the input dtype (e_natten/triton.py:515), so on 16-bit paths the backward's input is the
    rounded o; passing it here makes delta = dO.o use the same rounded values (rounding of an
    input is not an error of the backward).  None uses the exact o.
    """
    B, N, H, W, C = q.shape
    Hkv = k.shape[2]
    ks = kernel_size
    q, k, v, d_o = (t.to(acc_dtype) for t in (q, k, v, d_o))
    o_exact, lse = natten2d_fwd(q, k, v, ks, acc_dtype, rows, scale)
    delta = (d_o * (o_exact if o is None else o.to(acc_dtype))).sum(-1)
    wsx, wsy = _row_origins(H, ks, rows), window_start_table(W, ks)
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k).view(B, N, Hkv * W, C)
    dv = torch.zeros_like(k).view(B, N, Hkv * W, C)
    for u in range(ks):
        for w in range(ks):
            ku = _shifted(k, wsx, wsy, u, w)
            vu = _shifted(v, wsx, wsy, u, w)
            p = torch.exp(scale * (q * ku).sum(-1) - lse)
            ds = scale * p * ((d_o * vu).sum(-1) - delta)
            dq += ds.unsqueeze(-1) * ku
            lin = ((wsx + u).unsqueeze(1) * W + (wsy + w).unsqueeze(0)).reshape(-1)
            dk.index_add_(2, lin, (ds.unsqueeze(-1) * q).view(B, N, H * W, C))
            dv.index_add_(2, lin, (p.unsqueeze(-1) * d_o).view(B, N, H * W, C))
    return dq, dk.view(B, N, Hkv, W, C), dv.view(B, N, Hkv, W, C)


def natten2d_fwd_bwd(q, k, v, d_o, kernel_size: int, acc_dtype=torch.float64, rows=None, save_dtype=None,
                     scale: float = 1.0):
    """(o, lse, dq, dk, dv) in one call.  ``save_dtype``: dtype in which o is handed to the
    backward (the input dtype of a 16-bit path); None hands over the exact o."""
    o, lse = natten2d_fwd(q, k, v, kernel_size, acc_dtype, rows, scale)
    o_saved = None if save_dtype is None else o.to(save_dtype)
    dq, dk, dv = natten2d_bwd(q, k, v, d_o, kernel_size, acc_dtype, rows, o=o_saved, scale=scale)
    return o, lse, dq, dk, dv


# --------------------------------------------------------------------------- 1D operator
def natten1d_pixel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel_size: int) -> torch.Tensor:
    """Differentiable per-token loop on (B, N, T, C): for every token the kernel_size keys at
    the clamped origin, one softmax row (e_natten/pytorch.py:78-83 without the tiling)."""
    T = q.shape[2]
    outs = []
    for i in range(T):
        o0 = window_start(i, T, kernel_size)
        s = torch.matmul(q[:, :, i:i + 1, :], k[:, :, o0:o0 + kernel_size, :].transpose(-1, -2))
        outs.append(torch.matmul(torch.softmax(s, dim=-1), v[:, :, o0:o0 + kernel_size, :]))
    return torch.cat(outs, dim=2)


def natten1d_fwd(q, k, v, kernel_size: int, acc_dtype=torch.float64, scale: float = 1.0):
    """1D forward, vectorised over the window offsets.  Returns (o, lse) in ``acc_dtype``."""
    T = q.shape[2]
    q, k, v = q.to(acc_dtype) * scale, k.to(acc_dtype), v.to(acc_dtype)
    ws = window_start_table(T, kernel_size)
    s = torch.stack([(q * k.index_select(2, ws + u)).sum(-1) for u in range(kernel_size)])
    m = s.max(dim=0).values
    e = torch.exp(s - m)
    l = e.sum(0)
    o = sum((e[u] / l).unsqueeze(-1) * v.index_select(2, ws + u) for u in range(kernel_size))
    return o, m + torch.log(l)


def natten1d_bwd(q, k, v, d_o, kernel_size: int, acc_dtype=torch.float64, scale: float = 1.0):
    """1D backward in flash form.  Returns (dq, dk, dv) in ``acc_dtype``."""
    T = q.shape[2]
    q, k, v, d_o = (t.to(acc_dtype) for t in (q, k, v, d_o))
    o, lse = natten1d_fwd(q, k, v, kernel_size, acc_dtype, scale)
    delta = (d_o * o).sum(-1)
    ws = window_start_table(T, kernel_size)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    for u in range(kernel_size):
        ku, vu = k.index_select(2, ws + u), v.index_select(2, ws + u)
        p = torch.exp(scale * (q * ku).sum(-1) - lse)
        ds = scale * p * ((d_o * vu).sum(-1) - delta)
        dq += ds.unsqueeze(-1) * ku
        dk.index_add_(2, ws + u, ds.unsqueeze(-1) * q)
        dv.index_add_(2, ws + u, p.unsqueeze(-1) * d_o)
    return dq, dk, dv


# --------------------------------------------------------------------------- unfused pair
def natten2d_qk(q, k, kernel_size: int, acc_dtype=torch.float64):
    """Window scores (B, N, H, W, ks*ks): member j = (row j // ks, column j % ks) of the clamped
    window.  Differentiable."""
    B, N, H, W, C = q.shape
    ks = kernel_size
    q, k = q.to(acc_dtype), k.to(acc_dtype)
    wsx, wsy = window_start_table(H, ks), window_start_table(W, ks)
    return torch.stack([(q * _shifted(k, wsx, wsy, u, w)).sum(-1) for u in range(ks) for w in range(ks)], dim=-1)


def natten2d_av(attn, v, kernel_size: int, acc_dtype=torch.float64):
    """Applies window weights (B, N, H, W, ks*ks) to the values.  Differentiable."""
    B, N, H, W, C = v.shape
    ks = kernel_size
    attn, v = attn.to(acc_dtype), v.to(acc_dtype)
    wsx, wsy = window_start_table(H, ks), window_start_table(W, ks)
    return sum(attn[..., u * ks + w].unsqueeze(-1) * _shifted(v, wsx, wsy, u, w) for u in range(ks) for w in range(ks))


def round_inputs(shape, dtype, seed: int, scale: float = 1.0, q_scale: float = 1.0):
    """Seeded synthetic q, k, v, dO: drawn in fp32 on the CPU in that order from one
    generator, scaled, then rounded to ``dtype`` so that the oracle and the GPU see the
    same bits."""
    g = torch.Generator().manual_seed(seed)
    q, k, v, d_o = (torch.randn(shape, generator=g, dtype=torch.float32) * scale for _ in range(4))
    q = q * q_scale
    return tuple(t.to(dtype) for t in (q, k, v, d_o))
