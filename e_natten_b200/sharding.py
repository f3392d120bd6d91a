"""Multi-GPU use of the fused 2D neighborhood attention.

Two ways to split the work over the GPUs of one box, one process per GPU:

* **units** -- (batch, head) pairs are independent (every program of the reference touches only
  its own (b, n) slab, e_natten/triton.py:236-241).  ``partition_units`` gives each rank a
  contiguous range; no communication is needed.

* **rows of one huge image** -- rank r owns image rows ``[row0, row0 + R)``.  A query near the
  edge of its band looks at keys up to ``kernel_size // 2`` rows inside the neighbour's band, so
  before the forward each rank receives those K / V rows from its neighbours (the halo) and
  after the backward it sends the partial dK / dV it computed for those rows back to their
  owner, who adds them.  Only nearest neighbours talk, with point-to-point transfers through
  ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).  Received rows always land in this
  rank's own memory before a kernel reads them.  The kernels clamp windows against the whole
  image through a row view (``na2d_rows``), so the result equals the single-GPU result.

The arithmetic is injected (``forward_fn`` / ``backward_fn``) so that the exchange logic can be
exercised on CPU tensors in tests; by default it is the library's CUDA entry points.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import functional as F


def partition_units(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous split of ``n_units`` independent units: returns (first, count) for ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world / rank")
    base, extra = divmod(n_units, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def _window_start(i: int, seq_len: int, ks: int) -> int:
    return F.get_window_start(i, seq_len, ks)


@dataclass(frozen=True)
class RowShard:
    """Which rows of an H-row image a rank owns and which key rows its queries can see."""
    rank: int
    world: int
    H: int
    ks: int
    row0: int       # first owned row
    R: int          # owned rows
    kv_row0: int    # first key row any owned query sees
    Hkv: int        # key rows seen

    @property
    def top(self) -> int:          # halo rows owned by rank - 1
        return self.row0 - self.kv_row0

    @property
    def bot(self) -> int:          # halo rows owned by rank + 1
        return self.kv_row0 + self.Hkv - (self.row0 + self.R)

    def rows(self):
        return F.make_rows(self.row0, self.R, self.kv_row0, self.Hkv, self.H)


def plan_row_shard(H: int, world: int, rank: int, ks: int) -> RowShard:
    """Even split of H rows over ``world`` ranks.  Every band must be at least ``ks`` rows tall,
    so that a halo never reaches past the immediate neighbour."""
    first, count = partition_units(H, world, rank)
    if H // world < ks:
        raise ValueError(f"row bands of {H // world} rows are shorter than kernel_size {ks}")
    kv0 = _window_start(first, H, ks)
    kv1 = _window_start(first + count - 1, H, ks) + ks
    return RowShard(rank, world, H, ks, first, count, kv0, kv1 - kv0)


def _p2p(ops):
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()


def exchange_kv_halo(k_local: torch.Tensor, v_local: torch.Tensor, shard: RowShard,
                     group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns K and V extended by the halo rows of the neighbouring bands:
    shape (B, N, top + R + bot, W, C)."""
    B, N, R, W, C = k_local.shape
    assert R == shard.R
    up = plan_row_shard(shard.H, shard.world, shard.rank - 1, shard.ks) if shard.rank > 0 else None
    dn = plan_row_shard(shard.H, shard.world, shard.rank + 1, shard.ks) if shard.rank + 1 < shard.world else None
    ext = [t.new_empty((B, N, shard.Hkv, W, C)) for t in (k_local, v_local)]
    for e, t in zip(ext, (k_local, v_local)):
        e[:, :, shard.top:shard.top + R] = t
    ops, staged = [], []
    for e, t in zip(ext, (k_local, v_local)):
        if up is not None:
            if up.bot > 0:                                     # my first rows are rank-1's bottom halo
                send = t[:, :, :up.bot].contiguous()
                ops.append(dist.P2POp(dist.isend, send, shard.rank - 1, group))
            if shard.top > 0:
                recv = t.new_empty((B, N, shard.top, W, C))
                ops.append(dist.P2POp(dist.irecv, recv, shard.rank - 1, group))
                staged.append((e, slice(0, shard.top), recv))
        if dn is not None:
            if dn.top > 0:                                     # my last rows are rank+1's top halo
                send = t[:, :, R - dn.top:].contiguous()
                ops.append(dist.P2POp(dist.isend, send, shard.rank + 1, group))
            if shard.bot > 0:
                recv = t.new_empty((B, N, shard.bot, W, C))
                ops.append(dist.P2POp(dist.irecv, recv, shard.rank + 1, group))
                staged.append((e, slice(shard.top + R, shard.Hkv), recv))
    _p2p(ops)
    for e, sl, recv in staged:
        e[:, :, sl] = recv
    return ext[0], ext[1]


def reduce_dkdv_halo(dk_ext: torch.Tensor, dv_ext: torch.Tensor, shard: RowShard,
                     group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The matching reduction of the backward: partial dK / dV computed here for the neighbours'
    rows go back to their owners; partials the neighbours computed for this band's edge rows are
    added (in fp32, rounded once).  Returns dK, dV of shape (B, N, R, W, C)."""
    B, N, Hkv, W, C = dk_ext.shape
    R = shard.R
    up = plan_row_shard(shard.H, shard.world, shard.rank - 1, shard.ks) if shard.rank > 0 else None
    dn = plan_row_shard(shard.H, shard.world, shard.rank + 1, shard.ks) if shard.rank + 1 < shard.world else None
    ops, adds = [], []
    for e in (dk_ext, dv_ext):
        if up is not None:
            if shard.top > 0:                                  # rows I computed that rank-1 owns
                ops.append(dist.P2POp(dist.isend, e[:, :, :shard.top].contiguous(), shard.rank - 1, group))
            if up.bot > 0:                                     # rank-1's partials for my first rows
                recv = e.new_empty((B, N, up.bot, W, C))
                ops.append(dist.P2POp(dist.irecv, recv, shard.rank - 1, group))
                adds.append((e, slice(shard.top, shard.top + up.bot), recv))
        if dn is not None:
            if shard.bot > 0:
                ops.append(dist.P2POp(dist.isend, e[:, :, shard.top + R:].contiguous(), shard.rank + 1, group))
            if dn.top > 0:
                recv = e.new_empty((B, N, dn.top, W, C))
                ops.append(dist.P2POp(dist.irecv, recv, shard.rank + 1, group))
                adds.append((e, slice(shard.top + R - dn.top, shard.top + R), recv))
    _p2p(ops)
    for e, sl, recv in adds:
        acc = torch.promote_types(e.dtype, torch.float32)
        e[:, :, sl] = (e[:, :, sl].to(acc) + recv.to(acc)).to(e.dtype)
    return (dk_ext[:, :, shard.top:shard.top + R].contiguous(),
            dv_ext[:, :, shard.top:shard.top + R].contiguous())


def _default_forward(q, k_ext, v_ext, ks, rows):
    return F.natten2d_forward(q, k_ext, v_ext, ks, rows=rows)


def _default_backward(q, k_ext, v_ext, o, lse, d_o, ks, rows):
    return F.natten2d_backward(q, k_ext, v_ext, o, lse, d_o, ks, rows=rows)


class RowShardedNatten2d(torch.autograd.Function):
    """``natten2d`` on one row band of an image that is split over the ranks of ``group``."""

    @staticmethod
    def forward(ctx, q, k, v, kernel_size, shard: RowShard, group, forward_fn, backward_fn):
        k_ext, v_ext = exchange_kv_halo(k.contiguous(), v.contiguous(), shard, group)
        o, lse = (forward_fn or _default_forward)(q.contiguous(), k_ext, v_ext, kernel_size, shard.rows())
        ctx.save_for_backward(q, k_ext, v_ext, o, lse)
        ctx.kernel_size, ctx.shard, ctx.group, ctx.backward_fn = kernel_size, shard, group, backward_fn
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k_ext, v_ext, o, lse = ctx.saved_tensors
        d_q, dk_ext, dv_ext = (ctx.backward_fn or _default_backward)(
            q.contiguous(), k_ext, v_ext, o, lse, grad_output.contiguous(), ctx.kernel_size, ctx.shard.rows())
        d_k, d_v = reduce_dkdv_halo(dk_ext, dv_ext, ctx.shard, ctx.group)
        return d_q, d_k, d_v, None, None, None, None, None


def natten2d_row_sharded(q, k, v, kernel_size: int, H_global: int, group=None,
                         forward_fn: Optional[Callable] = None, backward_fn: Optional[Callable] = None):
    """Differentiable neighborhood attention over this rank's row band ``(B, N, R, W, C)`` of an
    image of ``H_global`` rows split evenly (``plan_row_shard``) over the ranks of ``group``."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    shard = plan_row_shard(H_global, world, rank, kernel_size)
    if q.shape[2] != shard.R:
        raise ValueError(f"rank {rank} must hold {shard.R} rows, got {q.shape[2]}")
    return RowShardedNatten2d.apply(q, k, v, kernel_size, shard, group, forward_fn, backward_fn)
