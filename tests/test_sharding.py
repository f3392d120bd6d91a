"""CPU tests (gloo, world size 2 and 3) of the multi-GPU host logic: unit partition, row-band
plan, K/V halo exchange and dK/dV halo reduction.  The arithmetic of each band is supplied by the
CPU oracle, so what is under test is the exchange itself: the bands must reassemble to the
whole-image result."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from e_natten_b200 import sharding
from oracle import na2d_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_units_covers_everything_once():
    for n in (1, 7, 16, 128, 256):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.partition_units(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (a, ca), (b, _) in zip(spans, spans[1:]):
                assert a + ca == b
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


def test_row_shard_plan_matches_window_union():
    for H, world, ks in ((1024, 8, 13), (1024, 2, 13), (48, 3, 5), (40, 2, 7), (39, 3, 13)):
        covered = 0
        for r in range(world):
            sh = sharding.plan_row_shard(H, world, r, ks)
            assert sh.row0 == covered
            covered += sh.R
            lo = min(orc.window_start(x, H, ks) for x in range(sh.row0, sh.row0 + sh.R))
            hi = max(orc.window_start(x, H, ks) + ks for x in range(sh.row0, sh.row0 + sh.R))
            assert (sh.kv_row0, sh.kv_row0 + sh.Hkv) == (lo, hi)
            assert 0 <= sh.top <= ks // 2 and 0 <= sh.bot <= ks // 2
            assert (sh.top == 0) == (r == 0) and (sh.bot == 0) == (r == world - 1)
        assert covered == H
    with pytest.raises(ValueError):
        sharding.plan_row_shard(20, 4, 0, 7)          # bands of 5 rows < kernel size


def _oracle_forward(q, k_ext, v_ext, ks, rows):
    o, lse = orc.natten2d_fwd(q, k_ext, v_ext, ks, rows=(rows.q_row0, rows.kv_row0, rows.H_global))
    return o.to(q.dtype), lse.float()


def _oracle_backward(q, k_ext, v_ext, o, lse, d_o, ks, rows):
    dq, dk, dv = orc.natten2d_bwd(q, k_ext, v_ext, d_o, ks, rows=(rows.q_row0, rows.kv_row0, rows.H_global))
    return dq.to(q.dtype), dk.to(q.dtype), dv.to(q.dtype)


def _worker(rank, world, port, H, W, ks, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        q, k, v, d_o = orc.round_inputs((1, 2, H, W, 3), torch.float64, 17)
        sh = sharding.plan_row_shard(H, world, rank, ks)
        band = slice(sh.row0, sh.row0 + sh.R)
        ql, kl, vl = (t[:, :, band].clone().requires_grad_() for t in (q, k, v))
        o = sharding.natten2d_row_sharded(ql, kl, vl, ks, H, forward_fn=_oracle_forward, backward_fn=_oracle_backward)
        o.backward(d_o[:, :, band])
        ro, _, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
        err = max((o.detach() - ro[:, :, band]).abs().max().item(),
                  (ql.grad - rdq[:, :, band]).abs().max().item(),
                  (kl.grad - rdk[:, :, band]).abs().max().item(),
                  (vl.grad - rdv[:, :, band]).abs().max().item())
        errs = [None] * world
        dist.all_gather_object(errs, err)
        if rank == 0:
            result.put(max(errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H,W,ks", [(2, 20, 9, 5), (3, 40, 14, 13), (2, 26, 14, 13), (3, 24, 7, 7)])
def test_row_sharded_bands_equal_whole_image(world, H, W, ks):
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, H, W, ks, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=5) < 1e-12


def _lonely_worker(rank, world, port, result):
    """Rank 1 leaves before the exchange; rank 0 must get an error from its bounded wait, not hang."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    # generous rendezvous (a loaded host can start the two processes seconds apart), short waits for
    # the exchange itself
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    group = dist.new_group(timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        os._exit(0)                                   # a rank that never takes part in the exchange
    q, k, v, _ = orc.round_inputs((1, 1, 20, 8, 2), torch.float64, 3)
    sh = sharding.plan_row_shard(20, world, rank, 5)
    band = slice(sh.row0, sh.row0 + sh.R)
    try:
        sharding.exchange_kv_halo(k[:, :, band].contiguous(), v[:, :, band].contiguous(), sh, group)
        result.put("no error")
    except Exception as exc:                          # noqa: BLE001 - any error from the transport is the point
        result.put("error: " + type(exc).__name__)
    os._exit(0)


def test_missing_neighbour_is_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lonely_worker, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=200)
    assert all(not p.is_alive() for p in procs)
    assert result.get(timeout=5).startswith("error")


def _subgroup_worker(rank, world, port, result):
    """The shard ranks live in a sub-group whose members are global ranks 1 and 2 (not 0 and 1):
    the point-to-point peers must be translated from group ranks to global ranks.  Rank 0 of the
    job does not take part.  A workspace keeps the extended K / V across two steps."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        group = dist.new_group(ranks=[1, 2])
        err = 0.0
        if rank >= 1:
            H, W, ks = 22, 9, 7
            q, k, v, d_o = orc.round_inputs((2, 1, H, W, 3), torch.float64, 29)
            sh = sharding.plan_row_shard(H, 2, dist.get_rank(group), ks)
            band = slice(sh.row0, sh.row0 + sh.R)
            ws = sharding.RowShardWorkspace(sh, 2, 1, W, 3, torch.float64, "cpu")
            ro, _, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
            for step in range(2):
                ws.k_local.copy_(k[:, :, band])                 # K / V built in place: no copy inside the call
                ws.v_local.copy_(v[:, :, band])
                ql = q[:, :, band].clone().requires_grad_()
                kl, vl = ws.k_local.detach().requires_grad_(), ws.v_local.detach().requires_grad_()
                o = sharding.natten2d_row_sharded(ql, kl, vl, ks, H, group=group, forward_fn=_oracle_forward,
                                                  backward_fn=_oracle_backward, workspace=ws)
                o.backward(d_o[:, :, band])
                err = max(err, (o.detach() - ro[:, :, band]).abs().max().item(),
                          (ql.grad - rdq[:, :, band]).abs().max().item(),
                          (kl.grad - rdk[:, :, band]).abs().max().item(),
                          (vl.grad - rdv[:, :, band]).abs().max().item())
        errs = [None] * world
        dist.all_gather_object(errs, err)
        if rank == 0:
            result.put(max(errs))
    finally:
        dist.destroy_process_group()


def test_row_sharding_inside_a_subgroup_that_does_not_start_at_rank_0():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_subgroup_worker, args=(r, 3, port, result)) for r in range(3)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=5) < 1e-12


# ---- the band path the GPU runs (whole-tile strips, fp32 edge partials, overlapped exchanges) --------------
def _band_worker(rank, world, port, H, W, ks, result):
    """forward_band_into / backward_band_into with the three launches replaced by the CPU oracle: what
    is under test is which rows each launch gets, what travels, and how the edge strips are put
    back together."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        q, k, v, d_o = orc.round_inputs((1, 2, H, W, 3), torch.float64, 29)
        sh = sharding.plan_row_shard(H, world, rank, ks)
        band = slice(sh.row0, sh.row0 + sh.R)
        ws = sharding.RowShardWorkspace(sh, 1, 2, W, 3, torch.float64, "cpu")
        ws.k_local.copy_(k[:, :, band])
        ws.v_local.copy_(v[:, :, band])
        calls = []

        def view(rows):
            return (rows.q_row0, rows.kv_row0, rows.H_global)

        def forward_into(qv, k_ext, v_ext, o, lse, kernel_size, rows=None, path="auto", scale=1.0, sm_margin=0):
            calls.append(("fwd", rows.q_row0 - sh.row0, rows.Hq, sm_margin))
            ro, rl = orc.natten2d_fwd(qv, k_ext, v_ext, kernel_size, rows=view(rows))
            o.copy_(ro)
            lse.copy_(rl)

        def backward_dq_into(qv, k_ext, v_ext, o, lse, g, d_q, delta, kernel_size, rows=None, path="auto", scale=1.0):
            dq, _, _ = orc.natten2d_bwd(qv, k_ext, v_ext, g, kernel_size, rows=view(rows))
            d_q.copy_(dq)

        def backward_dkdv_into(qv, k_sub, v_sub, lse, g, delta, d_k, d_v, kernel_size, rows=None, path="auto",
                               scale=1.0, sm_margin=0):
            # the key band of this call is a part of the extended rows: take that part of the full result
            lo = rows.kv_row0 - sh.kv_row0
            calls.append(("dkdv", lo, rows.Hkv, sm_margin))
            full = sharding.F.make_rows(sh.row0, sh.R, sh.kv_row0, sh.Hkv, sh.H)
            _, dk, dv = orc.natten2d_bwd(qv, ws.k_ext, ws.v_ext, g, kernel_size, rows=view(full))
            d_k.copy_(dk[:, :, lo:lo + rows.Hkv])
            d_v.copy_(dv[:, :, lo:lo + rows.Hkv])

        sharding.F.forward_into = forward_into
        sharding.F.backward_dq_into = backward_dq_into
        sharding.F.backward_dkdv_into = backward_dkdv_into
        ql, gl = q[:, :, band].contiguous(), d_o[:, :, band].contiguous()
        o = torch.empty_like(ql)
        lse = torch.empty(ql.shape[:4], dtype=torch.float32)
        sharding.forward_band_into(ws, ql, o, lse, ks)
        d_q, d_k, d_v = (torch.full_like(ql, float("nan")) for _ in range(3))
        delta = torch.empty_like(lse)
        sharding.backward_band_into(ws, ql, o, lse, gl, d_q, d_k, d_v, delta, ks)
        ro, _, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
        err = max((o - ro[:, :, band]).abs().max().item(), (d_q - rdq[:, :, band]).abs().max().item(),
                  (d_k - rdk[:, :, band]).abs().max().item(), (d_v - rdv[:, :, band]).abs().max().item())
        out = [None] * world
        dist.all_gather_object(out, (err, calls))
        if rank == 0:
            result.put(out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H,W,ks,whole_tiles", [(3, 144, 9, 7, True), (3, 60, 8, 5, False), (2, 96, 14, 13, True)])
def test_band_path_strips_and_partials_reassemble(world, H, W, ks, whole_tiles):
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_band_worker, args=(r, world, port, H, W, ks, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    out = result.get(timeout=5)
    assert max(e for e, _ in out) < 1e-12
    R = H // world
    for rank, (_, calls) in enumerate(out):
        fwd = [c for c in calls if c[0] == "fwd"]
        dkdv = [c for c in calls if c[0] == "dkdv"]
        sides = (rank > 0) + (rank < world - 1)
        assert len(fwd) == 1 + sides and len(dkdv) == 1 + sides
        # the launch that runs beside an exchange leaves SMs free; the strips after it do not
        assert fwd[0][3] > 0 and all(c[3] == 0 for c in fwd[1:])
        assert sum(c[2] for c in fwd) == R                       # every query row exactly once
        if whole_tiles:
            assert all(c[2] == 16 for c in fwd[1:])              # whole-tile strips
            assert all(c[2] == 16 for c in dkdv[:-1])
        elif sides == 2:
            assert all(c[2] == ks // 2 for c in fwd[1:])         # a band too short for two whole-tile strips
