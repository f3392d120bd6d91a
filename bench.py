#!/usr/bin/env python
"""Benchmark of the fused 2D neighborhood attention hot path (forward + backward).

    python bench.py --gpus N --steps K --warmup W [--workload c2-256] [--impl reference]

One step = one forward + one backward (dQ kernel, dK/dV kernel) over one batch of seeded
synthetic input that is already resident in HBM.  Work is split over GPUs by batch x head units
with no collective: every rank runs the same per-GPU workload (weak scaling) and the reported
value is the whole job's throughput, units of all ranks / max-over-ranks time.

The printed JSON line carries
  value / ms_per_step   effective TFLOP/s of forward+backward (FLOPs = 4*B*N*H*W*ks^2*C forward,
                        2.5x that backward) on resident inputs, CUDA-event timed,
  e2e                   the same metric through the public autograd entry point with pinned HOST
                        buffers: host->device copies of q, k, v, dO and device->host copies of
                        o, dQ, dK, dV inside the timed region, pipelined over slices of the
                        (batch, head) units on three streams,
  roofline              the dominant kernel against the measured HBM peak (MEASURED_PEAKS.json),
  roofline_step         the whole step's algorithmic bytes (12T + 2L) against the same peak,
  cpu_baseline          the CPU oracle port timed on this host on a bounded sample,
  clocks                SM clocks and throttle reasons sampled through NVML during the timed region.

`--impl reference` times the CPU port of the reference's algorithm (oracle/) on the host cores,
since the reference itself is Python that needs its source checkout and a Triton-capable
GPU path that does not exist for bf16 backward; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> (B, N, H, W, C, ks, dtype, seed, scale, q_scale)
WORKLOADS = {
    "c1": (1, 2, 16, 16, 32, 5, "fp32", 0, 1.0, 1.0),
    "c2-32": (4, 4, 32, 32, 128, 5, "bf16", 0, 1.0, 128 ** -0.5),
    "c2-64": (4, 4, 64, 64, 128, 5, "bf16", 0, 1.0, 128 ** -0.5),
    "c2-128": (4, 4, 128, 128, 128, 5, "bf16", 0, 1.0, 128 ** -0.5),
    "c2-192": (4, 4, 192, 192, 128, 5, "bf16", 0, 1.0, 128 ** -0.5),
    "c2-256": (4, 4, 256, 256, 128, 5, "bf16", 0, 1.0, 128 ** -0.5),      # the headline
    "c3": (32, 2, 56, 56, 32, 7, "bf16", 1, 0.5, 1.0),
    "c4a": (16, 8, 28, 28, 64, 13, "bf16", 2, 1.0, 1.0),
    "c4b": (16, 16, 14, 14, 64, 13, "bf16", 2, 1.0, 1.0),
    "c5": (1, 8, 1024, 1024, 128, 13, "bf16", 3, 1.0, 1.0),
    "c5-256": (1, 8, 256, 256, 128, 13, "bf16", 3, 1.0, 1.0),           # c5 at a size an ncu capture can hold
}
FALLBACK_HBM_GBS = 6650.0


def flops_fwd(B, N, H, W, C, ks):
    return 4.0 * B * N * H * W * ks * ks * C


def algorithmic_bytes(B, N, H, W, C, esize):
    T = B * N * H * W * C * esize
    L = B * N * H * W * 4
    return {"fwd": 4 * T + L, "dq": 6 * T + 2 * L, "dkdv": 6 * T + 2 * L, "bwd": 8 * T + L,
            "step": 12 * T + 2 * L, "T": T, "L": L}


# DRAM bytes (read + written) per launch, per byte of one (B, N, H, W, C) tensor, from one ncu
# capture of workload c2 at side 128 (profiles/tcgen05_fwd_dq_dkdv_c2_bf16.md).  Reads equal the
# input bytes, so the traffic of the other c2 sides follows in proportion to the tensor size.
NCU_DRAM_BYTES_PER_TENSOR_BYTE = {"na2d forward": 3.652, "na2d backward dQ": 4.786, "na2d backward dK/dV": 5.554}
NCU_TRAFFIC_SOURCE = "ncu capture of c2-128 scaled by tensor bytes"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 0.0))), "measured"
    return FALLBACK_HBM_GBS, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only queries) from a
    background thread, every few milliseconds, between start() and stop()."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
               "sw_power_cap": 0x4}

    def __init__(self, uuid: str, period_s: float = 0.004):
        self.uuid, self.period = uuid, period_s
        self.samples, self.max_mhz, self.err = [], None, None
        self._stop = threading.Event()
        self._thread = None
        self._window = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:                      # no NVML: report that, never guess
            self.err = f"NVML unavailable: {exc}"
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                self.samples.append((time.perf_counter(), float(mhz), int(mask)))
            except Exception as exc:
                self.err = str(exc)
                return
            time.sleep(self.period)

    def mark(self, t0: float, t1: float):
        """Host-clock window of the timed region; only samples inside it are reported."""
        self._window = (t0, t1)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self.err and not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0, "reasons": [self.err]}
        sel = self.samples
        if self._window:
            sel = [x for x in self.samples if self._window[0] <= x[0] <= self._window[1]]
        reasons = sorted(n for n, bit in self.REASONS.items() if any(x[2] & bit for x in sel))
        return {"sm_mhz": statistics.median(x[1] for x in sel) if sel else None, "sm_max_mhz": self.max_mhz,
                "samples": len(sel), "reasons": reasons}


# --------------------------------------------------------------------------------------- CPU arm
def cpu_port_sample(wl, budget_s: float, threads: int):
    """Time the oracle port (forward + backward, fp32 accumulation) on a row band of one
    (batch, head) unit of the workload, sized from a short calibration to about `budget_s`
    seconds.  Returns (seconds, flops_of_sample, description)."""
    import torch
    from oracle import na2d_oracle as orc
    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    torch.set_num_threads(threads)
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dtype]

    def run(rows_q):
        rows_q = max(1, min(H, rows_q))
        a = max(0, (H - rows_q) // 2)
        e = a + rows_q
        kv0 = orc.window_start(a, H, ks)
        kv1 = orc.window_start(e - 1, H, ks) + ks
        g = torch.Generator().manual_seed(seed)
        mk = lambda r: (torch.randn((1, 1, r, W, C), generator=g, dtype=torch.float32) * scale).to(dt)
        q, d_o = mk(rows_q) * q_scale, mk(rows_q)
        k, v = mk(kv1 - kv0), mk(kv1 - kv0)
        t0 = time.perf_counter()
        orc.natten2d_fwd_bwd(q.to(dt), k, v, d_o, ks, acc_dtype=torch.float32, rows=(a, kv0, H))
        return time.perf_counter() - t0, rows_q

    t_cal, r_cal = run(min(H, 8))
    rows = int(max(r_cal, min(H, r_cal * budget_s / max(t_cal, 1e-4))))
    t, rows = run(rows)
    fl = 3.5 * flops_fwd(1, 1, rows, W, C, ks)
    return t, fl, f"rows [{(H - rows) // 2},{(H - rows) // 2 + rows}) of one (batch, head) unit, all {W} columns"


def run_reference_arm(args, wl_name, wl):
    """The reference's algorithm on the host cores (CPU port in oracle/): one bounded sample per
    step.  Under a multi-rank launch only rank 0 works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch
    B, N, H, W, C, ks, dtype, *_ = wl
    threads = os.cpu_count() or 1
    per_step = max(0.5, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_port_sample(wl, per_step, threads)
    times, fl, what = [], 0.0, ""
    for _ in range(args.steps):
        t, fl, what = cpu_port_sample(wl, per_step, threads)
        times.append(t)
    t_mean = sum(times) / len(times)
    val = fl / t_mean / 1e12
    line = {
        "impl": "reference", "metric": "effective_tflops_fwd_bwd", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "B": B, "heads": N, "H": H, "W": W, "head_dim": C, "kernel_size": ks,
                   "input_dtype": dtype, "sample_per_step": what},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": what},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- row-sharded arm
def run_row_sharded(args, wl, dev, rank, world):
    """One huge image split by rows over the ranks (strong scaling): every step exchanges the
    kernel_size//2-row K/V halo with the neighbours, runs forward + backward on the band through
    a row view, and reduces the dK/dV halo.  Device-timed, max over ranks."""
    import torch
    import torch.distributed as dist
    import e_natten_b200 as na
    from e_natten_b200 import functional as F, sharding

    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    sh = sharding.plan_row_shard(H, world, rank, ks)
    g = torch.Generator(device=dev).manual_seed(seed + 1000 * rank)
    mk = lambda: (torch.randn((B, N, sh.R, W, C), generator=g, device=dev, dtype=torch.float32) * scale).to(dt)
    q, k, v, d_o = mk(), mk(), mk(), mk()
    o, d_q = torch.empty_like(q), torch.empty_like(q)
    lse = torch.empty((B, N, sh.R, W), dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)
    rows = sh.rows()

    def step():
        k_ext, v_ext = sharding.exchange_kv_halo(k, v, sh)
        F.forward_into(q, k_ext, v_ext, o, lse, ks, rows=rows)
        dk_ext, dv_ext = torch.empty_like(k_ext), torch.empty_like(v_ext)
        F.backward_dq_into(q, k_ext, v_ext, o, lse, d_o, d_q, delta, ks, rows=rows)
        F.backward_dkdv_into(q, k_ext, v_ext, lse, d_o, delta, dk_ext, dv_ext, ks, rows=rows)
        return sharding.reduce_dkdv_halo(dk_ext, dv_ext, sh)

    for _ in range(args.warmup):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    na.check_kernels(dev)
    launches0 = na.launch_count()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        step()
    t1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([t0.elapsed_time(t1) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    if rank == 0:
        fl = 3.5 * flops_fwd(B, N, H, W, C, ks)
        esize = torch.empty((), dtype=dt).element_size()
        ab = algorithmic_bytes(B, N, H, W, C, esize)
        hbm_peak, _, peak_kind = measured_peaks()
        halo = 2 * (ks // 2) * W * C * esize * B * N       # one tensor, both sides of an interior band
        print(json.dumps({
            "metric": "effective_tflops_fwd_bwd", "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "heads": N, "H": H, "W": W, "head_dim": C, "kernel_size": ks,
                       "sharding": f"rows, {sh.R} per GPU, {ks // 2}-row K/V halo exchange + dK/dV halo reduction (NCCL p2p)",
                       "halo_bytes_per_step_per_gpu": 4 * halo, "l2": "inputs larger than L2"},
            "roofline_step": {"bound": "hbm", "achieved": ab["step"] / world / (ms * 1e-3) / 1e9, "peak": hbm_peak,
                              "unit": "GB/s", "frac": ab["step"] / world / (ms * 1e-3) / 1e9 / hbm_peak,
                              "peak_source": peak_kind},
            "gpu_launches": na.launch_count() - launches0}), flush=True)
    dist.destroy_process_group()


# --------------------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2-256", choices=sorted(WORKLOADS))
    ap.add_argument("--dtype", default=None, choices=[None, "bf16", "fp16", "fp32"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = list(WORKLOADS[args.workload])
    if args.dtype:
        wl[6] = args.dtype
    wl = tuple(wl)

    if args.impl == "reference":
        run_reference_arm(args, args.workload, wl)
        return

    import torch
    import torch.distributed as dist
    import e_natten_b200 as na
    from e_natten_b200 import functional as F

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.workload == "c5" and world > 1:        # the single huge image is split by rows
        run_row_sharded(args, wl, dev, rank, world)
        return

    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
    esize = torch.empty((), dtype=dt).element_size()
    shape = (B, N, H, W, C)

    # Seeded synthetic inputs, drawn on the device per rank (each rank has its own units).
    g = torch.Generator(device=dev).manual_seed(seed + 1000 * rank)
    mk = lambda: (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * scale)
    q = (mk() * q_scale).to(dt)
    k, v, d_o = mk().to(dt), mk().to(dt), mk().to(dt)
    o, d_q, d_k, d_v = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((B, N, H, W), dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)
    ab = algorithmic_bytes(B, N, H, W, C, esize)
    resident = 8 * ab["T"] + 2 * ab["L"]
    flush = None
    if resident < 512 << 20:          # working set not well above L2: flush it between steps
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step(events=None):
        if flush is not None:
            flush.fill_(1)
        if events:
            events[0].record()
        F.forward_into(q, k, v, o, lse, ks, path=args.path)
        if events:
            events[1].record()
        F.backward_dq_into(q, k, v, o, lse, d_o, d_q, delta, ks, path=args.path)
        if events:
            events[2].record()
        F.backward_dkdv_into(q, k, v, lse, d_o, delta, d_k, d_v, ks, path=args.path)
        if events:
            events[3].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    na.check_kernels(dev)

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    launches0 = na.launch_count()
    barrier()
    t_host0 = time.perf_counter()
    for i in range(args.steps):
        step(evs[i])
    barrier()
    sampler.mark(t_host0, time.perf_counter())
    launches = na.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    na.check_kernels(dev)

    fwd_ms = [e[0].elapsed_time(e[1]) for e in evs]
    dq_ms = [e[1].elapsed_time(e[2]) for e in evs]
    dkdv_ms = [e[2].elapsed_time(e[3]) for e in evs]
    step_ms = [e[0].elapsed_time(e[3]) for e in evs]
    mean = lambda xs: sum(xs) / len(xs)
    t = torch.tensor([mean(step_ms), mean(fwd_ms), mean(dq_ms), mean(dkdv_ms)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step, ms_fwd, ms_dq, ms_dkdv = t.tolist()

    # ---- end to end through the public entry point with host buffers --------------------------
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hg = (x.to("cpu").pin_memory() for x in (q, k, v, d_o))
        ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
        n_e2e = max(2, min(args.steps, 5))

        # The step is pipelined over slices of the (batch x head) units, as a user with host data
        # would do it: slice j+1 is copied in and slice j-1 copied out (PCIe is full duplex) while
        # slice j runs through natten2d + backward.
        units = B * N
        n_sl = 8 if units % 8 == 0 else (units if units <= 8 else 1)
        u = units // n_sl
        hin = [x.view(units, 1, H, W, C) for x in (hq, hk, hv, hg)]
        hout = [x.view(units, 1, H, W, C) for x in (ho, hdq, hdk, hdv)]
        dev_in = [[torch.empty((u, 1, H, W, C), dtype=q.dtype, device=dev) for _ in range(4)] for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

        def e2e_step():
            cur = torch.cuda.current_stream()
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            ready = [torch.cuda.Event() for _ in range(n_sl)]
            done = [torch.cuda.Event() for _ in range(n_sl)]
            for j in range(n_sl):
                sl = slice(j * u, (j + 1) * u)
                slot = dev_in[j % 2]
                with torch.cuda.stream(s_in):
                    if j >= 2:
                        s_in.wait_event(done[j - 2])          # the slot's previous slice has been consumed
                    for dst, src in zip(slot, hin):
                        dst.copy_(src[sl], non_blocking=True)
                    ready[j].record(s_in)
                cur.wait_event(ready[j])
                dq_, dk_, dv_ = (t.detach().requires_grad_() for t in slot[:3])
                out = na.natten2d(dq_, dk_, dv_, ks)
                out.backward(slot[3])
                done[j].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done[j])
                    for hdst, src in zip(hout, (out.detach(), dq_.grad, dk_.grad, dv_.grad)):
                        hdst[sl].copy_(src, non_blocking=True)
                        src.record_stream(s_out)
            cur.wait_stream(s_out)

        e2e_step()
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(n_e2e):
            e2e_step()
        t1.record()
        barrier()
        te = torch.tensor([t0.elapsed_time(t1) / n_e2e], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = te.item()
        # the host buffers of the last pipelined step must hold what the resident-input step produced
        for name, host, devt in (("o", ho, o), ("dQ", hdq, d_q), ("dK", hdk, d_k), ("dV", hdv, d_v)):
            if not torch.equal(host[-1, -1], devt[-1, -1].cpu()) or not torch.equal(host[0, 0], devt[0, 0].cpu()):
                raise RuntimeError(f"end-to-end path: host {name} differs from the resident-input result")
        e2e = {"value": 3.5 * flops_fwd(*shape, ks) * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "ms_per_step": e2e_ms, "h2d_bytes_per_step": 4 * ab["T"], "d2h_bytes_per_step": 4 * ab["T"],
               "pipeline": f"{n_sl} slices of {u} (batch, head) units; copy-in, natten2d + backward and copy-out on three streams"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    fl_step = 3.5 * flops_fwd(*shape, ks)
    kern = {"na2d forward": (ms_fwd, ab["fwd"]), "na2d backward dQ": (ms_dq, ab["dq"]),
            "na2d backward dK/dV": (ms_dkdv, ab["dkdv"])}
    dom = max(kern, key=lambda n: kern[n][0])
    dom_ms, dom_bytes = kern[dom]
    traffic = None
    if args.workload.startswith("c2-") and dtype in ("bf16", "fp16") and args.path != "simt":
        traffic = NCU_DRAM_BYTES_PER_TENSOR_BYTE[dom] * ab["T"]
    ach = dom_bytes / (dom_ms * 1e-3) / 1e9
    step_ach = ab["step"] / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "effective_tflops_fwd_bwd", "value": fl_step * world / (ms_step * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == "fp32" else dtype, "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "heads": N, "H": H, "W": W, "head_dim": C,
                   "kernel_size": ks, "input_dtype": dtype, "accumulate": "fp32", "path": args.path,
                   "units_per_gpu": B * N, "sharding": "batch x head units, no collective",
                   "l2": "inputs larger than L2" if flush is None else "L2 flushed between steps (256 MiB write)"},
        "fwd_ms": ms_fwd, "bwd_dq_ms": ms_dq, "bwd_dkdv_ms": ms_dkdv,
        "fwd_tflops": flops_fwd(*shape, ks) / (ms_fwd * 1e-3) / 1e12,
        "bwd_tflops": 2.5 * flops_fwd(*shape, ks) / ((ms_dq + ms_dkdv) * 1e-3) / 1e12,
        "tensor_roofline_frac": fl_step / (ms_step * 1e-3) / 1e12 / tensor_peak if tensor_peak else None,
        "roofline": {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                     "frac": ach / hbm_peak, "traffic": traffic,
                     "traffic_source": NCU_TRAFFIC_SOURCE if traffic else None, "peak_source": peak_kind,
                     "algorithmic_bytes_per_launch": dom_bytes},
        "roofline_step": {"bound": "hbm", "achieved": step_ach, "peak": hbm_peak, "unit": "GB/s",
                          "frac": step_ach / hbm_peak, "algorithmic_bytes": ab["step"]},
        "gpu_launches": launches, "clocks": clocks,
    }
    if e2e:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        t_cpu, fl_cpu, what = cpu_port_sample(wl, 15.0, threads)
        line["cpu_baseline"] = {"value": fl_cpu / t_cpu / 1e12, "unit": "TFLOP/s", "cores": threads,
                                "kind": "port", "sample": what, "seconds": t_cpu}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
