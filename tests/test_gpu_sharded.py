"""GPU test of the row-sharded path on two GPUs (skipped where fewer are visible): each rank runs
its band of one image through the halo exchange, the CUDA kernels with a row view and the dK/dV
halo reduction over NCCL; the bands must equal the whole-image result computed on one GPU."""
import datetime
import os
import socket
import sys
import time
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_close, make_inputs

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, shape, ks, dtype, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120),
                            device_id=dev)
    try:
        import e_natten_b200 as na
        from e_natten_b200 import sharding
        q, k, v, d_o = make_inputs(shape, dtype, 23, q_scale=shape[-1] ** -0.5)
        H = shape[2]
        sh = sharding.plan_row_shard(H, world, rank, ks)
        band = slice(sh.row0, sh.row0 + sh.R)
        ql, kl, vl = (t[:, :, band].to(dev).requires_grad_() for t in (q, k, v))
        o = sharding.natten2d_row_sharded(ql, kl, vl, ks, H)
        o.backward(d_o[:, :, band].to(dev))
        na.check_kernels(dev)
        # whole image on this rank's GPU for comparison
        qw, kw, vw = (t.to(dev).requires_grad_() for t in (q, k, v))
        ow = na.natten2d(qw, kw, vw, ks)
        ow.backward(d_o.to(dev))
        ok = True
        try:
            assert_close(o, ow[:, :, band].double(), dtype, "o band")
            assert_close(ql.grad, qw.grad[:, :, band].double(), dtype, "dq band")
            assert_close(kl.grad, kw.grad[:, :, band].double(), dtype, "dk band")
            assert_close(vl.grad, vw.grad[:, :, band].double(), dtype, "dv band")
        except AssertionError as exc:
            ok = str(exc)
        oks = [None] * world
        dist.all_gather_object(oks, ok)
        if rank == 0:
            result.put(oks)
    except BaseException:
        # leave at once and loudly: the parent sees the exit code and stops the other rank, which
        # may be waiting for a transfer from this one; tearing the process group down here could block
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)
    dist.destroy_process_group()


@pytest.mark.parametrize("shape,ks,dtype", [((1, 2, 64, 40, 64), 7, torch.bfloat16),
                                            ((1, 2, 48, 24, 128), 13, torch.float16),
                                            ((2, 2, 40, 24, 128), 5, torch.bfloat16),     # strip kernels
                                            ((1, 2, 36, 40, 64), 3, torch.float16)])
def test_row_sharded_two_gpus(shape, ks, dtype):
    _run_world(2, shape, ks, dtype)


@pytest.mark.parametrize("shape,ks,dtype", [((1, 2, 144, 24, 64), 7, torch.bfloat16),      # whole-tile strips on both sides
                                            ((1, 2, 60, 40, 128), 5, torch.bfloat16)])     # bands too short for them
def test_row_sharded_three_gpus_middle_rank_has_two_neighbours(shape, ks, dtype):
    _run_world(3, shape, ks, dtype)


def _run_world(world, shape, ks, dtype):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, shape, ks, dtype, result)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.time() + 240
    while any(p.is_alive() for p in procs) and time.time() < deadline:
        if any(p.exitcode not in (None, 0) for p in procs):
            break
        time.sleep(0.2)
    for p in procs:
        if p.is_alive():                     # never leave a stuck rank behind: pytest would wait for it at exit
            p.kill()
        p.join()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert result.get(timeout=5) == [True] * world
