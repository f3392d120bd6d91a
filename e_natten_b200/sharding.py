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

  How a step runs (``RowShardedNatten2d``):

  - K and V live in *extended* buffers ``(B, N, top + R + bot, W, C)`` whose middle rows are the
    rank's own; a caller that builds K / V directly in ``RowShardWorkspace.k_local`` / ``v_local``
    pays no copy, any other K / V is copied into the middle once.
  - The halo rows are received straight into the first / last rows of the extended buffers, one
    contiguous run per (batch, head) slab, while the forward of the *interior* query rows - those
    whose windows stay inside the rank's own rows - already runs; the two boundary strips of
    ``kernel_size // 2`` query rows follow when the halo has arrived.
  - The backward computes dQ for the band, and dK / dV in up to three launches over parts of the
    extended key rows: the interior key rows go straight into dK / dV; the two edge strips (halo
    rows and the own rows the neighbours' queries also see) are partial sums and are kept in fp32
    (a partial sum can be much larger than the total, so it is not rounded to 16 bits before it
    is added); the halo rows' partials go to their owners while the interior launch runs, and
    what arrives is added to the own edge rows and rounded once.

The arithmetic is injected (``forward_fn`` / ``backward_fn``) so that the exchange logic can be
exercised on CPU tensors in tests; by default it is the library's CUDA entry points.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import os

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

    def rows(self, a: int = 0, b: Optional[int] = None):
        """Row view of the local query rows [a, b) (default: the whole band) over the extended keys."""
        b = self.R if b is None else b
        return F.make_rows(self.row0 + a, b - a, self.kv_row0, self.Hkv, self.H)


def plan_row_shard(H: int, world: int, rank: int, ks: int) -> RowShard:
    """Even split of H rows over ``world`` ranks.  Every band must be at least ``ks`` rows tall,
    so that a halo never reaches past the immediate neighbour."""
    first, count = partition_units(H, world, rank)
    if H // world < ks:
        raise ValueError(f"row bands of {H // world} rows are shorter than kernel_size {ks}")
    kv0 = _window_start(first, H, ks)
    kv1 = _window_start(first + count - 1, H, ks) + ks
    return RowShard(rank, world, H, ks, first, count, kv0, kv1 - kv0)


def _neighbours(shard: RowShard):
    up = plan_row_shard(shard.H, shard.world, shard.rank - 1, shard.ks) if shard.rank > 0 else None
    dn = plan_row_shard(shard.H, shard.world, shard.rank + 1, shard.ks) if shard.rank + 1 < shard.world else None
    return up, dn


def _peer(group, group_rank: int) -> int:
    """The rank ``dist.P2POp`` wants: global, while a shard's rank counts inside ``group``."""
    return group_rank if group is None else dist.get_global_rank(group, group_rank)


def _partial_dtype(dtype: torch.dtype) -> torch.dtype:
    """dtype in which partial dK / dV travel and are added."""
    return torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype


_TILE_ROWS = 16      # rows of a kernel tile: launches over whole tiles waste no tile rows


def _up16(n: int) -> int:
    return (n + _TILE_ROWS - 1) // _TILE_ROWS * _TILE_ROWS


def _query_strips(shard: RowShard) -> Tuple[int, int]:
    """(a, b): the band's query rows [a, b) run before the halo has arrived, [0, a) and [b, R)
    after it.  Rows [0, top) and [R - bot, R) are the ones that need halo rows; the strips are
    widened to whole tiles where the band is tall enough, so that the three launches together
    cover no more tile rows than one launch over the band would."""
    R, a, b = shard.R, shard.top, shard.bot
    wa, wb = (_up16(a) if a else 0), (_up16(b) if b else 0)
    if wa + wb <= R:
        a, b = wa, wb
    return a, R - b


def _key_strips(shard: RowShard) -> Tuple[int, int, int, int]:
    """(own_top, own_bot, n_up, n_dn): the key half's top strip covers the upper halo rows and
    the first own_top own rows, its bottom strip the last own_bot own rows and the lower halo rows;
    the neighbours' partials arrive for the first n_up and the last n_dn own rows (own_top >= n_up,
    own_bot >= n_dn).  The strips are widened to whole tiles where the band is tall enough."""
    up, dn = _neighbours(shard)
    n_up = up.bot if up is not None else 0
    n_dn = dn.top if dn is not None else 0
    own_top, own_bot = n_up, n_dn
    wt = _up16(shard.top + n_up) - shard.top if shard.top + n_up > 0 else 0
    wb = _up16(shard.bot + n_dn) - shard.bot if shard.bot + n_dn > 0 else 0
    if wt + wb <= shard.R:
        own_top, own_bot = wt, wb
    return own_top, own_bot, n_up, n_dn


class RowShardWorkspace:
    """The buffers of one rank that outlive a step: extended K / V (own rows in the middle, halo
    rows around them), and the fp32 extended dK / dV with the receive buffers of their reduction.
    ``k_local`` / ``v_local`` are views of the middle rows: K / V written there need no copy."""

    def __init__(self, shard: RowShard, B: int, N: int, W: int, C: int, dtype: torch.dtype, device,
                 sm_margin: Optional[int] = None):
        self.shard = shard
        # SMs the launches that run beside an exchange leave to NCCL's copy kernels: the persistent
        # kernels otherwise hold every SM (and nearly all of its shared memory) until they end, and
        # the transfer that was meant to run under them runs after them
        if sm_margin is None:
            sm_margin = int(os.environ.get("NA2D_SHARD_SM_MARGIN", "16"))
        self.sm_margin = sm_margin if shard.world > 1 else 0
        shape = (B, N, shard.Hkv, W, C)
        self.k_ext = torch.empty(shape, dtype=dtype, device=device)
        self.v_ext = torch.empty(shape, dtype=dtype, device=device)
        self._partial = None
        self._shape, self._dtype, self._device = shape, dtype, device

    @property
    def k_local(self) -> torch.Tensor:
        return self.k_ext[:, :, self.shard.top:self.shard.top + self.shard.R]

    @property
    def v_local(self) -> torch.Tensor:
        return self.v_ext[:, :, self.shard.top:self.shard.top + self.shard.R]

    def matches(self, k: torch.Tensor) -> bool:
        return tuple(k.shape) == tuple(self.k_local.shape) and k.dtype == self._dtype and k.device == self.k_ext.device

    def edge_buffers(self):
        """fp32 buffers of the two edge strips of the key half (halo rows plus the own rows the
        neighbours contribute to), [dK, dV] each, and the receive buffers of the neighbours'
        partials; allocated on first use."""
        if getattr(self, "_edges", None) is None:
            sh = self.shard
            B, N, _, W, C = self._shape
            pd = _partial_dtype(self._dtype)
            own_top, own_bot, n_up, n_dn = _key_strips(sh)
            mk = lambda rows: [torch.empty((B, N, rows, W, C), dtype=pd, device=self._device) for _ in range(2)] if rows > 0 else None
            self._edges = {"top": mk(sh.top + own_top), "bot": mk(sh.bot + own_bot), "recv_up": mk(n_up), "recv_dn": mk(n_dn)}
        return self._edges

    def partial_buffers(self):
        """(dk_ext, dv_ext, recv_up, recv_dn): fp32 (or the inputs' wider dtype), allocated on first use."""
        if self._partial is None:
            sh = self.shard
            B, N, _, W, C = self._shape
            pd = _partial_dtype(self._dtype)
            up, dn = _neighbours(sh)
            mk = lambda rows: torch.empty((2, B, N, rows, W, C), dtype=pd, device=self._device) if rows > 0 else None
            self._partial = (torch.empty(self._shape, dtype=pd, device=self._device),
                             torch.empty(self._shape, dtype=pd, device=self._device),
                             mk(up.bot if up is not None else 0), mk(dn.top if dn is not None else 0))
        return self._partial


def _slabs(t: torch.Tensor, rows: slice) -> List[torch.Tensor]:
    """The contiguous per-(batch, head) runs of rows ``rows`` of a (B, N, rows, W, C) tensor."""
    B, N = t.shape[:2]
    return [t[b, n, rows] for b in range(B) for n in range(N)]


def start_kv_halo_exchange(k_ext: torch.Tensor, v_ext: torch.Tensor, shard: RowShard, group=None):
    """Starts the halo exchange of the extended K / V buffers (own rows already in the middle):
    sends this rank's edge rows to the neighbours that see them and receives the halo rows straight
    into the buffers' first / last rows.  Returns the pending requests; ``finish_exchange`` waits."""
    up, dn = _neighbours(shard)
    top, R = shard.top, shard.R
    ops = []
    for e in (k_ext, v_ext):
        if up is not None:
            if up.bot > 0:                                     # my first rows are rank-1's bottom halo
                ops += [dist.P2POp(dist.isend, s, _peer(group, shard.rank - 1), group)
                        for s in _slabs(e, slice(top, top + up.bot))]
            if top > 0:
                ops += [dist.P2POp(dist.irecv, s, _peer(group, shard.rank - 1), group) for s in _slabs(e, slice(0, top))]
        if dn is not None:
            if dn.top > 0:                                     # my last rows are rank+1's top halo
                ops += [dist.P2POp(dist.isend, s, _peer(group, shard.rank + 1), group)
                        for s in _slabs(e, slice(top + R - dn.top, top + R))]
            if shard.bot > 0:
                ops += [dist.P2POp(dist.irecv, s, _peer(group, shard.rank + 1), group)
                        for s in _slabs(e, slice(top + R, shard.Hkv))]
    return dist.batch_isend_irecv(ops) if ops else []


def finish_exchange(reqs) -> None:
    for req in reqs:
        req.wait()


def exchange_kv_halo(k_local: torch.Tensor, v_local: torch.Tensor, shard: RowShard,
                     group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Blocking form for callers without a workspace: returns K and V extended by the halo rows of
    the neighbouring bands, shape (B, N, top + R + bot, W, C)."""
    B, N, R, W, C = k_local.shape
    assert R == shard.R
    ext = [t.new_empty((B, N, shard.Hkv, W, C)) for t in (k_local, v_local)]
    for e, t in zip(ext, (k_local, v_local)):
        e[:, :, shard.top:shard.top + R] = t
    finish_exchange(start_kv_halo_exchange(ext[0], ext[1], shard, group))
    return ext[0], ext[1]


def reduce_dkdv_halo(dk_ext: torch.Tensor, dv_ext: torch.Tensor, shard: RowShard, group=None,
                     out_dtype: Optional[torch.dtype] = None, recv=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The matching reduction of the backward: partial dK / dV computed here for the neighbours'
    rows go back to their owners; partials the neighbours computed for this band's edge rows are
    added, in the partials' dtype (fp32 for 16-bit tensors), and the sum is rounded once to
    ``out_dtype``.  Returns dK, dV of shape (B, N, R, W, C)."""
    B, N, Hkv, W, C = dk_ext.shape
    R, top = shard.R, shard.top
    up, dn = _neighbours(shard)
    n_up = up.bot if up is not None else 0
    n_dn = dn.top if dn is not None else 0
    recv_up, recv_dn = recv if recv is not None else (None, None)
    if n_up > 0 and recv_up is None:
        recv_up = dk_ext.new_empty((2, B, N, n_up, W, C))
    if n_dn > 0 and recv_dn is None:
        recv_dn = dk_ext.new_empty((2, B, N, n_dn, W, C))
    ops = []
    for i, e in enumerate((dk_ext, dv_ext)):
        if up is not None:
            if top > 0:                                        # rows I computed that rank-1 owns
                ops += [dist.P2POp(dist.isend, s, _peer(group, shard.rank - 1), group) for s in _slabs(e, slice(0, top))]
            if n_up > 0:                                       # rank-1's partials for my first rows
                ops += [dist.P2POp(dist.irecv, s, _peer(group, shard.rank - 1), group)
                        for s in _slabs(recv_up[i], slice(0, n_up))]
        if dn is not None:
            if shard.bot > 0:
                ops += [dist.P2POp(dist.isend, s, _peer(group, shard.rank + 1), group)
                        for s in _slabs(e, slice(top + R, Hkv))]
            if n_dn > 0:
                ops += [dist.P2POp(dist.irecv, s, _peer(group, shard.rank + 1), group)
                        for s in _slabs(recv_dn[i], slice(0, n_dn))]
    finish_exchange(dist.batch_isend_irecv(ops) if ops else [])
    outs = []
    for i, e in enumerate((dk_ext, dv_ext)):
        local = e[:, :, top:top + R]
        if n_up > 0:
            local[:, :, :n_up] += recv_up[i]
        if n_dn > 0:
            local[:, :, R - n_dn:] += recv_dn[i]
        outs.append(local.to(out_dtype or e.dtype).contiguous())
    return outs[0], outs[1]


def forward_band_into(ws: RowShardWorkspace, q, o, lse, kernel_size: int, group=None, scale: float = 1.0,
                      path: str = "auto") -> None:
    """Forward of this rank's band into caller-owned ``o`` (B, N, R, W, C) and ``lse`` (B, N, R, W),
    K / V already in ``ws.k_local`` / ``ws.v_local``: starts the halo exchange, runs the interior
    query rows meanwhile and the two boundary strips once the halo is there.  No autograd."""
    sh = ws.shard
    reqs = start_kv_halo_exchange(ws.k_ext, ws.v_ext, sh, group)
    a, b = _query_strips(sh)
    spans = [(a, b)]

    def run(lo, hi, sm_margin=0):
        part = torch.empty(lse.shape[:2] + (hi - lo, lse.shape[3]), dtype=torch.float32, device=lse.device)
        F.forward_into(q[:, :, lo:hi], ws.k_ext, ws.v_ext, o[:, :, lo:hi], part, kernel_size, rows=sh.rows(lo, hi),
                       path=path, scale=scale, sm_margin=sm_margin)
        return part

    parts = [run(a, b, ws.sm_margin if reqs else 0)]
    finish_exchange(reqs)
    if a > 0:
        spans.append((0, a))
        parts.append(run(0, a))
    if b < sh.R:
        spans.append((b, sh.R))
        parts.append(run(b, sh.R))
    for (lo, hi), part in zip(spans, parts):
        lse[:, :, lo:hi].copy_(part)


def backward_band_into(ws: RowShardWorkspace, q, o, lse, d_o, d_q, d_k, d_v, delta, kernel_size: int, group=None,
                       scale: float = 1.0, path: str = "auto") -> None:
    """Backward of this rank's band into caller-owned ``d_q``, ``d_k``, ``d_v`` (B, N, R, W, C).

    dQ comes from one launch over the band.  The key half runs in up to three launches over parts
    of the extended key rows: the interior key rows - every query that sees them is local - go
    straight into ``d_k`` / ``d_v`` in the tensors' dtype; the two edge strips (the halo rows this
    rank computed for its neighbours, and its own rows next to them - at least those the neighbours'
    queries see as well, widened to a whole tile of rows where the band is tall enough) go into
    small fp32 buffers.  The halo partials are sent to their owners, what arrives is added to the
    own edge rows, and those are rounded once into ``d_k`` / ``d_v``.  The interior launch, which
    runs while the partials travel, leaves ``ws.sm_margin`` SMs to the transfer."""
    sh = ws.shard
    up, dn = _neighbours(sh)
    top, bot, R = sh.top, sh.bot, sh.R
    own_top, own_bot, n_up, n_dn = _key_strips(sh)
    F.backward_dq_into(q, ws.k_ext, ws.v_ext, o, lse, d_o, d_q, delta, kernel_size, rows=sh.rows(), path=path, scale=scale)
    edges = ws.edge_buffers()

    def key_half(ext_lo, ext_hi, dk, dv, sm_margin=0):
        rows = F.make_rows(sh.row0, R, sh.kv_row0 + ext_lo, ext_hi - ext_lo, sh.H)
        F.backward_dkdv_into(q, ws.k_ext[:, :, ext_lo:ext_hi], ws.v_ext[:, :, ext_lo:ext_hi], lse, d_o, delta, dk, dv,
                             kernel_size, rows=rows, path=path, scale=scale, sm_margin=sm_margin)

    # edge strips first, so that their partials are on their way while the interior runs
    if top + own_top > 0:
        key_half(0, top + own_top, edges["top"][0], edges["top"][1])
    if bot + own_bot > 0:
        key_half(top + R - own_bot, sh.Hkv, edges["bot"][0], edges["bot"][1])
    ops = []
    for i in range(2):
        if up is not None:
            if top > 0:
                ops += [dist.P2POp(dist.isend, s, _peer(group, sh.rank - 1), group) for s in _slabs(edges["top"][i], slice(0, top))]
            if n_up > 0:
                ops += [dist.P2POp(dist.irecv, s, _peer(group, sh.rank - 1), group) for s in _slabs(edges["recv_up"][i], slice(0, n_up))]
        if dn is not None:
            if bot > 0:
                ops += [dist.P2POp(dist.isend, s, _peer(group, sh.rank + 1), group)
                        for s in _slabs(edges["bot"][i], slice(own_bot, own_bot + bot))]
            if n_dn > 0:
                ops += [dist.P2POp(dist.irecv, s, _peer(group, sh.rank + 1), group) for s in _slabs(edges["recv_dn"][i], slice(0, n_dn))]
    reqs = dist.batch_isend_irecv(ops) if ops else []
    if R - own_top - own_bot > 0:
        key_half(top + own_top, top + R - own_bot, d_k[:, :, own_top:R - own_bot], d_v[:, :, own_top:R - own_bot],
                 ws.sm_margin if reqs else 0)
    finish_exchange(reqs)
    for i, out in enumerate((d_k, d_v)):
        if own_top > 0:
            own = edges["top"][i][:, :, top:]                       # the strip's own rows, fp32
            if n_up > 0:
                own[:, :, :n_up] += edges["recv_up"][i]
            out[:, :, :own_top] = own
        if own_bot > 0:
            own = edges["bot"][i][:, :, :own_bot]
            if n_dn > 0:
                own[:, :, own_bot - n_dn:] += edges["recv_dn"][i]
            out[:, :, R - own_bot:] = own


def _default_forward(q, k_ext, v_ext, ks, rows):
    return F.natten2d_forward(q, k_ext, v_ext, ks, rows=rows)


def _default_backward(q, k_ext, v_ext, o, lse, d_o, ks, rows):
    return F.natten2d_backward(q, k_ext, v_ext, o, lse, d_o, ks, rows=rows, dkdv_dtype=_partial_dtype(q.dtype))


class RowShardedNatten2d(torch.autograd.Function):
    """``natten2d`` on one row band of an image that is split over the ranks of ``group``."""

    @staticmethod
    def forward(ctx, q, k, v, kernel_size, shard: RowShard, group, forward_fn, backward_fn, workspace):
        fwd = forward_fn or _default_forward
        B, N, R, W, C = q.shape
        ws = workspace
        if ws is None or not ws.matches(k):
            ws = RowShardWorkspace(shard, B, N, W, C, k.dtype, k.device)
        for ext_local, t in ((ws.k_local, k), (ws.v_local, v)):
            if t.data_ptr() != ext_local.data_ptr() or t.stride() != ext_local.stride():
                ext_local.copy_(t)                     # K / V built elsewhere: one copy into the middle rows
        reqs = start_kv_halo_exchange(ws.k_ext, ws.v_ext, shard, group)
        # interior query rows see no halo row: their forward runs while the halo is on its way
        a, b = _query_strips(shard)
        parts = [None, fwd(q[:, :, a:b], ws.k_ext, ws.v_ext, kernel_size, shard.rows(a, b)), None]
        finish_exchange(reqs)
        if a > 0:
            parts[0] = fwd(q[:, :, :a], ws.k_ext, ws.v_ext, kernel_size, shard.rows(0, a))
        if b < R:
            parts[2] = fwd(q[:, :, b:], ws.k_ext, ws.v_ext, kernel_size, shard.rows(b, R))
        parts = [p for p in parts if p is not None]
        o = torch.cat([p[0] for p in parts], dim=2) if len(parts) > 1 else parts[0][0]
        lse = torch.cat([p[1] for p in parts], dim=2) if len(parts) > 1 else parts[0][1]
        ctx.save_for_backward(q, ws.k_ext, ws.v_ext, o, lse)
        ctx.kernel_size, ctx.shard, ctx.group, ctx.backward_fn, ctx.ws = kernel_size, shard, group, backward_fn, ws
        ctx.kv_dtype = k.dtype
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, k_ext, v_ext, o, lse = ctx.saved_tensors
        if ctx.backward_fn is None:               # the library's kernels: key half in interior + edge launches
            d_o = F.as_kernel_input(grad_output)
            d_q = torch.empty(q.shape, dtype=q.dtype, device=q.device)
            d_k = torch.empty(q.shape, dtype=ctx.kv_dtype, device=q.device)
            d_v = torch.empty(q.shape, dtype=ctx.kv_dtype, device=q.device)
            delta = torch.empty(lse.shape, dtype=torch.float32, device=q.device)
            backward_band_into(ctx.ws, F.as_kernel_input(q), o, lse, d_o, d_q, d_k, d_v, delta, ctx.kernel_size, ctx.group)
            return d_q, d_k, d_v, None, None, None, None, None, None
        d_q, dk_ext, dv_ext = (ctx.backward_fn or _default_backward)(
            q, k_ext, v_ext, o, lse, grad_output, ctx.kernel_size, ctx.shard.rows())
        pd = _partial_dtype(ctx.kv_dtype)
        if dk_ext.dtype != pd:                       # an injected backward that returns the tensors' dtype
            dk_ext, dv_ext = dk_ext.to(pd), dv_ext.to(pd)
        d_k, d_v = reduce_dkdv_halo(dk_ext, dv_ext, ctx.shard, ctx.group, out_dtype=ctx.kv_dtype)
        return d_q, d_k, d_v, None, None, None, None, None, None


def natten2d_row_sharded(q, k, v, kernel_size: int, H_global: int, group=None,
                         forward_fn: Optional[Callable] = None, backward_fn: Optional[Callable] = None,
                         workspace: Optional[RowShardWorkspace] = None):
    """Differentiable neighborhood attention over this rank's row band ``(B, N, R, W, C)`` of an
    image of ``H_global`` rows split evenly (``plan_row_shard``) over the ranks of ``group``.
    ``workspace`` (optional) keeps the extended K / V buffers across steps; K / V that are its
    ``k_local`` / ``v_local`` views are used in place."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    shard = plan_row_shard(H_global, world, rank, kernel_size)
    if q.shape[2] != shard.R:
        raise ValueError(f"rank {rank} must hold {shard.R} rows, got {q.shape[2]}")
    return RowShardedNatten2d.apply(q, k, v, kernel_size, shard, group, forward_fn, backward_fn, workspace)
