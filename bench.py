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
                        (batch, head) units on three streams; with the copy rates each rank gets
                        when it does nothing but copy (what the host side can deliver),
  roofline              the dominant kernel against the measured HBM peak (MEASURED_PEAKS.json),
  roofline_step         the whole step's algorithmic bytes (12T + 2L) against the same peak,
  cpu_baseline          the reference's own CPU code (e_natten.pytorch, staged under oracle/_ref) on
                        its CPU-runnable configuration, and the oracle port on a bounded sample
                        of the benched workload, both timed on this host,
  clocks                SM clocks and throttle reasons sampled through NVML during the timed region,
  extra.sweep           (1 GPU) every BASELINE configuration, bf16 and fp16, and the README shapes
                        in fp32, each forward / dQ / dK,dV / step,
  extra.strong          (N > 1) the headline workload's 16 units split over the N GPUs,
  extra.c5_row_sharded  (N > 1) the single huge image split by rows over the N GPUs with the K/V
                        halo exchange and the dK/dV halo reduction, against the same image on
                        one GPU.

`--impl reference` times the reference's own CPU implementation (e_natten.pytorch from
oracle/_ref; the oracle port where that file has not been staged) on the host cores, each step a
bounded sample of the workload; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
DTYPE_NAMES = {"fp32": "float32", "bf16": "bfloat16", "fp16": "float16"}


def flops_fwd(B, N, H, W, C, ks):
    return 4.0 * B * N * H * W * ks * ks * C


def algorithmic_bytes(B, N, H, W, C, esize):
    T = B * N * H * W * C * esize
    L = B * N * H * W * 4
    # per launch: forward reads q,k,v and writes o,lse; the dQ kernel reads q,k,v,dO,lse and writes dQ,delta;
    # the dK/dV kernel reads q,k,v,dO,lse,delta and writes dK,dV.  "bwd" and "step" are the one-pass figures.
    return {"fwd": 4 * T + L, "dq": 5 * T + 2 * L, "dkdv": 6 * T + 2 * L, "bwd": 8 * T + L,
            "step": 12 * T + 2 * L, "T": T, "L": L}


# DRAM bytes (read + written) per launch of the three kernels on the headline workload, from an ncu
# capture of that workload itself (dram__bytes_read.sum + dram__bytes_write.sum, one launch each).
NCU_DRAM_BYTES = {"c2-256": {"na2d forward": 806513920 + 248424448, "na2d backward dQ": 1088127232 + 250111744,
                             "na2d backward dK/dV": 1086513408 + 500653056}}
NCU_TRAFFIC_SOURCE = "ncu capture of this workload (c2-256), one launch per kernel"


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

    def __init__(self, uuid: str, period_s: float = 0.002):
        self.uuid, self.period = uuid, period_s
        self.samples, self.max_mhz, self.err = [], None, None
        self._stop = threading.Event()
        self._thread = None
        self._windows = {}

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

    def mark(self, name: str, t0: float, t1: float):
        """Host-clock window of a timed region; samples are reported per window."""
        self._windows.setdefault(name, []).append((t0, t1))

    def _summary(self, sel):
        reasons = sorted(n for n, bit in self.REASONS.items() if any(x[2] & bit for x in sel))
        return {"sm_mhz": statistics.median(x[1] for x in sel) if sel else None, "sm_max_mhz": self.max_mhz,
                "samples": len(sel), "reasons": reasons}

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if self.err and not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0, "reasons": [self.err]}
        inside = lambda name: [x for x in self.samples if any(a <= x[0] <= b for a, b in self._windows.get(name, []))]
        out = self._summary(inside("timed"))
        every = [x for x in self.samples if any(a <= x[0] <= b for ws in self._windows.values() for a, b in ws)]
        # the headline's timed region is a few tens of milliseconds; the other timed regions of the
        # same run (end to end, sweep) give the record under load that a sample count needs
        out["all_timed_regions"] = self._summary(every)
        if out["samples"] == 0 and every:
            # an NVML query takes milliseconds: a headline region of a few steps can end between two
            out.update({k: out["all_timed_regions"][k] for k in ("sm_mhz", "reasons")})
            out["window"] = "no sample fell inside the headline region; figures of all timed regions of this run"
        return out


# --------------------------------------------------------------------------------------- CPU arm
def cpu_port_sample(wl, budget_s: float, threads: int):
    """Time the oracle port (forward + backward, fp32 accumulation) on a row band of one
    (batch, head) unit of the workload, sized from a short calibration to about `budget_s`
    seconds.  Returns (seconds, flops_of_sample, description)."""
    import torch
    from oracle import na2d_oracle as orc
    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    torch.set_num_threads(threads)
    dt = getattr(torch, DTYPE_NAMES[dtype])

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
    return t, fl, f"oracle port, rows [{(H - rows) // 2},{(H - rows) // 2 + rows}) of one (batch, head) unit, all {W} columns"


def cpu_reference_sample(wl, budget_s: float, threads: int):
    """Time the reference's own CPU code - e_natten.pytorch.natten2d forward + .backward(dO), the
    file staged under oracle/_ref - on a small image with the workload's head dim and kernel size,
    fp32 (the dtype the reference is tested in), sized to about `budget_s` seconds.  Returns
    (seconds, nominal flops, description) or None if the file has not been staged.

    Caveat that goes with every number from this function: the reference's backward fills dQ for
    its first 3x3 tile only (e_natten/pytorch.py:228-231), so it does less than the nominal work;
    the flops counted are the nominal ones."""
    import torch
    from oracle import build_ref
    ref = build_ref.load()
    if ref is None:
        return None
    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    torch.set_num_threads(threads)

    def run(b, n, h, w):
        g = torch.Generator().manual_seed(seed)
        q, k, v, d_o = (torch.randn((b, n, h, w, C), generator=g, dtype=torch.float32) * scale for _ in range(4))
        q = (q * q_scale).requires_grad_()
        k.requires_grad_()
        v.requires_grad_()
        t0 = time.perf_counter()
        ref.natten2d(q, k, v, ks).backward(d_o)
        return time.perf_counter() - t0

    if B * N * H * W <= 1024:                        # the CPU-runnable configuration: run it whole
        t = run(B, N, H, W)
        return t, 3.5 * flops_fwd(B, N, H, W, C, ks), f"e_natten.pytorch.natten2d on the whole workload ({B}x{N}x{H}x{W}x{C}, fp32)"
    t_cal = run(1, 1, ks, ks + 3)
    per_px = t_cal / (ks * (ks + 3))
    w = int(max(ks + 3, min(W, budget_s / per_px / ks)))
    t = run(1, 1, ks, w)
    return t, 3.5 * flops_fwd(1, 1, ks, w, C, ks), (f"e_natten.pytorch.natten2d on a {ks}x{w} image of one (batch, head) unit, head dim {C}, "
                                                   f"kernel size {ks}, fp32: {ks * w} of the workload's {B * N * H * W} pixels")


def run_reference_arm(args, wl_name, wl):
    """The reference's CPU implementation on the host cores: one bounded sample per step.  Under a
    multi-rank launch only rank 0 works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    B, N, H, W, C, ks, dtype, *_ = wl
    threads = os.cpu_count() or 1
    per_step = max(0.5, min(20.0, 150.0 / max(1, args.steps + args.warmup)))
    sample = lambda: cpu_reference_sample(wl, per_step, threads)
    kind = "reference"
    if sample() is None:
        kind = "port"
        sample = lambda: cpu_port_sample(wl, per_step, threads)
    for _ in range(max(0, args.warmup - 1)):
        sample()
    times, fl, what = [], 0.0, ""
    for _ in range(args.steps):
        t, fl, what = sample()
        times.append(t)
    t_mean = sum(times) / len(times)
    val = fl / t_mean / 1e12
    line = {
        "impl": "reference", "metric": "effective_tflops_fwd_bwd", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "B": B, "heads": N, "H": H, "W": W, "head_dim": C, "kernel_size": ks,
                   "input_dtype": dtype, "sample_per_step": what},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": what},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if kind == "reference":
        line["cpu_baseline"]["note"] = ("the reference's backward fills dQ for its first 3x3 tile only "
                                        "(e_natten/pytorch.py:228-231); flops counted are the nominal ones")
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- GPU problems
class Problem:
    """Resident tensors of one workload on one GPU and its three launches."""

    def __init__(self, wl, dev, path, seed_offset=0, units=None):
        import torch
        from e_natten_b200 import functional as F
        self.F, self.torch = F, torch
        B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
        if units is not None:                        # a slice of the (batch, head) units
            B, N = units, 1
        self.shape, self.ks, self.path, self.dtype_name = (B, N, H, W, C), ks, path, dtype
        dt = getattr(torch, DTYPE_NAMES[dtype])
        self.esize = torch.empty((), dtype=dt).element_size()
        g = torch.Generator(device=dev).manual_seed(seed + seed_offset)
        mk = lambda: (torch.randn(self.shape, generator=g, device=dev, dtype=torch.float32) * scale)
        self.q = (mk() * q_scale).to(dt)
        self.k, self.v, self.d_o = mk().to(dt), mk().to(dt), mk().to(dt)
        self.o, self.d_q, self.d_k, self.d_v = (torch.empty_like(self.q) for _ in range(4))
        self.lse = torch.empty((B, N, H, W), dtype=torch.float32, device=dev)
        self.delta = torch.empty_like(self.lse)
        self.ab = algorithmic_bytes(B, N, H, W, C, self.esize)
        resident = 8 * self.ab["T"] + 2 * self.ab["L"]
        # working set not well above L2 (126 MB): flush it between steps
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if resident < 512 << 20 else None

    def step(self, events=None):
        F, ks, path = self.F, self.ks, self.path
        if self.flush is not None:
            self.flush.fill_(1)
        if events:
            events[0].record()
        F.forward_into(self.q, self.k, self.v, self.o, self.lse, ks, path=path)
        if events:
            events[1].record()
        F.backward_dq_into(self.q, self.k, self.v, self.o, self.lse, self.d_o, self.d_q, self.delta, ks, path=path)
        if events:
            events[2].record()
        F.backward_dkdv_into(self.q, self.k, self.v, self.lse, self.d_o, self.delta, self.d_k, self.d_v, ks, path=path)
        if events:
            events[3].record()

    def flops(self):
        return 3.5 * flops_fwd(*self.shape, self.ks)

    def time(self, steps, warmup, barrier=None):
        """CUDA-event times (ms, mean over `steps`) of forward, dQ, dK/dV and the whole step."""
        torch = self.torch
        for _ in range(max(warmup, 3)):
            self.step()
        (barrier or torch.cuda.synchronize)()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        t0 = time.perf_counter()
        for i in range(steps):
            self.step(evs[i])
        (barrier or torch.cuda.synchronize)()
        t1 = time.perf_counter()
        mean = lambda xs: sum(xs) / len(xs)
        return {"fwd_ms": mean([e[0].elapsed_time(e[1]) for e in evs]), "dq_ms": mean([e[1].elapsed_time(e[2]) for e in evs]),
                "dkdv_ms": mean([e[2].elapsed_time(e[3]) for e in evs]), "step_ms": mean([e[0].elapsed_time(e[3]) for e in evs]),
                "host_window": (t0, t1)}


def sweep_record(name, p, t, hbm_peak):
    B, N, H, W, C = p.shape
    return {"workload": name, "dtype": p.dtype_name, "shape": [B, N, H, W, C], "kernel_size": p.ks,
            "fwd_ms": round(t["fwd_ms"], 5), "bwd_dq_ms": round(t["dq_ms"], 5), "bwd_dkdv_ms": round(t["dkdv_ms"], 5),
            "ms_per_step": round(t["step_ms"], 5), "tflops": round(p.flops() / (t["step_ms"] * 1e-3) / 1e12, 3),
            "hbm_frac_step": round(p.ab["step"] / (t["step_ms"] * 1e-3) / 1e9 / hbm_peak, 4),
            "l2": "inputs larger than L2" if p.flush is None else "L2 flushed between steps"}


def run_sweep(dev, path, hbm_peak, sampler, free_bytes):
    """Every BASELINE configuration in bf16 and fp16, and the README shapes in fp32 (the dtype the
    reference benchmarks in, bench.py:19,44), a handful of steps each."""
    import gc
    import torch
    out = []
    plan = [("c1", None)]
    plan += [(f"c2-{s}", d) for s in (32, 64, 128, 192, 256) for d in ("bf16", "fp16")]
    plan += [("c3", "bf16"), ("c3", "fp16"), ("c4a", "bf16"), ("c4a", "fp16"), ("c4b", "bf16"), ("c4b", "fp16")]
    plan += [(f"c2-{s}", "fp32") for s in (32, 64, 128, 256)]
    plan += [("c5", "bf16")]
    for name, dtype in plan:
        wl = list(WORKLOADS[name])
        if dtype:
            wl[6] = dtype
        B, N, H, W, C = wl[:5]
        need = 10 * B * N * H * W * C * (4 if wl[6] == "fp32" else 2) + 3 * B * N * H * W * C * 4
        if need > free_bytes:
            out.append({"workload": name, "dtype": wl[6], "skipped": "not enough free device memory"})
            continue
        p = Problem(tuple(wl), dev, path)
        slow = wl[6] == "fp32" or name == "c5"
        t = p.time(3 if slow else 10, 3)
        sampler.mark("sweep", *t["host_window"])
        out.append(sweep_record(name, p, t, hbm_peak))
        del p
        gc.collect()
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------- row-sharded sub-record
def run_row_sharded(wl, dev, rank, world, steps, warmup):
    """One huge image split by rows over the ranks (strong scaling): every step starts the
    kernel_size//2-row K/V halo exchange, runs the interior rows' forward meanwhile and the boundary
    rows after it, then the backward on the band and the fp32 dK/dV halo reduction.  Device-timed,
    max over ranks.  Returns (ms per step, rows per GPU, halo bytes per step of an interior rank)."""
    import torch
    import torch.distributed as dist
    from e_natten_b200 import sharding

    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    dt = getattr(torch, DTYPE_NAMES[dtype])
    sh = sharding.plan_row_shard(H, world, rank, ks)
    ws = sharding.RowShardWorkspace(sh, B, N, W, C, dt, dev)
    g = torch.Generator(device=dev).manual_seed(seed + 1000 * rank)
    mk = lambda: (torch.randn((B, N, sh.R, W, C), generator=g, device=dev, dtype=torch.float32) * scale).to(dt)
    q, d_o = mk(), mk()
    ws.k_local.copy_(mk())                               # K / V are built in place, in the extended buffers
    ws.v_local.copy_(mk())
    o, d_q, d_k, d_v = (torch.empty_like(q) for _ in range(4))
    lse = torch.empty((B, N, sh.R, W), dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)

    def step():
        sharding.forward_band_into(ws, q, o, lse, ks)
        sharding.backward_band_into(ws, q, o, lse, d_o, d_q, d_k, d_v, delta, ks)

    for _ in range(max(warmup, 3)):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    t1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([t0.elapsed_time(t1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    esize = torch.empty((), dtype=dt).element_size()
    halo_rows = 2 * (ks // 2)
    halo_bytes = halo_rows * W * C * B * N * (2 * esize + 2 * 4)      # K, V in; fp32 dK, dV partials out
    return t.item(), sh.R, halo_bytes


# --------------------------------------------------------------------------------------- host side of a rank
def bind_to_gpu_numa_node(dev_index: int):
    """Run this process (and with it the pages it pins) on the CPUs of the NUMA node the GPU's PCIe
    port hangs off.  Read-only look-ups in sysfs plus sched_setaffinity on this process; nothing
    about the GPU or the host is changed.  Returns the node, or None where it cannot be told."""
    try:
        import torch
        props = torch.cuda.get_device_properties(dev_index)
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
        return node
    except Exception:                                  # no sysfs, no such attribute: stay where we are
        return None


def copy_rates(torch, dev, nbytes, barrier):
    """GB/s a rank gets from pinned host memory to the device and back when all ranks do nothing but
    copy at the same time (both directions at once, as the end-to-end pipeline does)."""
    host_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    host_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    for _ in range(2):                                  # the second round is the one reported
        barrier()
        with torch.cuda.stream(s1):
            ev[0].record()
            d_in.copy_(host_in, non_blocking=True)
            ev[1].record()
        with torch.cuda.stream(s2):
            ev[2].record()
            host_out.copy_(d_out, non_blocking=True)
            ev[3].record()
        barrier()
    return nbytes / (ev[0].elapsed_time(ev[1]) * 1e-3) / 1e9, nbytes / (ev[2].elapsed_time(ev[3]) * 1e-3) / 1e9


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
    ap.add_argument("--no-extra", action="store_true", help="skip the sweep / strong / row-sharded sub-records")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = list(WORKLOADS[args.workload])
    if args.dtype:
        wl[6] = args.dtype
    wl = tuple(wl)

    if args.impl == "reference":
        run_reference_arm(args, args.workload, wl)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    import gc
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU; there is no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_node = bind_to_gpu_numa_node(local_rank)       # before anything is pinned
    import e_natten_b200 as na
    from e_natten_b200 import sharding
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # point-to-point only; no multicast objects to bind
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    B, N, H, W, C, ks, dtype, seed, scale, q_scale = wl
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    prob = Problem(wl, dev, args.path, seed_offset=1000 * rank)
    ab, shape = prob.ab, prob.shape

    # ---- the timed region: exactly `steps` steps, device-timed, max over ranks ------------------------
    for _ in range(args.warmup):
        prob.step()
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
        prob.step(evs[i])
    barrier()
    sampler.mark("timed", t_host0, time.perf_counter())
    launches = na.launch_count() - launches0
    na.check_kernels(dev)
    mean = lambda xs: sum(xs) / len(xs)
    ms_step, ms_fwd, ms_dq, ms_dkdv = max_over_ranks([
        mean([e[0].elapsed_time(e[3]) for e in evs]), mean([e[0].elapsed_time(e[1]) for e in evs]),
        mean([e[1].elapsed_time(e[2]) for e in evs]), mean([e[2].elapsed_time(e[3]) for e in evs])])

    # ---- end to end through the public entry point with host buffers --------------------------
    e2e = None
    if not args.no_e2e:
        q, k, v, d_o = prob.q, prob.k, prob.v, prob.d_o
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
        th0 = time.perf_counter()
        t0.record()
        for _ in range(n_e2e):
            e2e_step()
        t1.record()
        barrier()
        sampler.mark("e2e", th0, time.perf_counter())
        e2e_ms = max_over_ranks([t0.elapsed_time(t1) / n_e2e])[0]
        # the host buffers of the last pipelined step must hold what the resident-input step produced
        for name, host, devt in (("o", ho, prob.o), ("dQ", hdq, prob.d_q), ("dK", hdk, prob.d_k), ("dV", hdv, prob.d_v)):
            if not torch.equal(host[-1, -1], devt[-1, -1].cpu()) or not torch.equal(host[0, 0], devt[0, 0].cpu()):
                raise RuntimeError(f"end-to-end path: host {name} differs from the resident-input result")
        # what the host side delivers to each rank when the ranks only copy (both directions at once)
        h2d, d2h = copy_rates(torch, dev, 256 << 20, barrier)
        rates = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        all_rates = [torch.zeros_like(rates) for _ in range(world)]
        nodes = [None] * world
        if world > 1:
            dist.all_gather(all_rates, rates)
            dist.all_gather_object(nodes, numa_node)
        else:
            all_rates, nodes = [rates], [numa_node]
        e2e = {"value": prob.flops() * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "ms_per_step": e2e_ms, "h2d_bytes_per_step": 4 * ab["T"], "d2h_bytes_per_step": 4 * ab["T"],
               "pipeline": f"{n_sl} slices of {u} (batch, head) units; copy-in, natten2d + backward and copy-out on three streams",
               "achieved_copy_gbs_per_rank_each_way": round(4 * ab["T"] / (e2e_ms * 1e-3) / 1e9, 2),
               "copy_only_gbs_per_rank": [{"rank": r, "numa_node": nodes[r], "h2d": round(x[0].item(), 2), "d2h": round(x[1].item(), 2)}
                                          for r, x in enumerate(all_rates)],
               "note": "copy_only = each rank copying 256 MiB each way at the same time as all other ranks, no kernels: "
                       "the rate the host side delivers; the pipelined step cannot be faster than its bytes at that rate"}
        del hq, hk, hv, hg, ho, hdq, hdk, hdv, dev_in, hin, hout

    # ---- sub-records ---------------------------------------------------------------------------
    extra = {}
    flops_step = prob.flops()
    if not args.no_extra and args.workload == "c2-256" and args.path == "auto" and not args.dtype:
        del prob
        gc.collect()
        torch.cuda.empty_cache()
        if world == 1:
            free_bytes, _ = torch.cuda.mem_get_info(dev)
            extra["sweep"] = run_sweep(dev, args.path, hbm_peak, sampler, int(free_bytes * 0.9))
        else:
            # strong scaling: the headline's 16 (batch, head) units split over the ranks
            first, count = sharding.partition_units(B * N, world, rank)
            sp = Problem(wl, dev, args.path, seed_offset=1000 * rank, units=max(count, 1))
            s_ms = max_over_ranks([sp.time(args.steps, args.warmup, barrier)["step_ms"]])[0]
            del sp
            gc.collect()
            torch.cuda.empty_cache()
            extra["strong"] = {"workload": "c2-256", "units_total": B * N, "units_per_gpu": (B * N + world - 1) // world,
                               "ms_per_step": s_ms, "value": 3.5 * flops_fwd(B, N, H, W, C, ks) / (s_ms * 1e-3) / 1e12,
                               "unit": "TFLOP/s", "scaling": "strong",
                               "note": "the 1-GPU line's ms_per_step divided by this is the strong-scaling speed-up"}
            # the single huge image: whole on one GPU (every rank measures it, max taken), then row-sharded
            c5 = WORKLOADS["c5"]
            one = Problem(c5, dev, args.path, seed_offset=1000 * rank)
            t1 = max_over_ranks([one.time(3, 3, barrier)["step_ms"]])[0]
            del one
            gc.collect()
            torch.cuda.empty_cache()
            tn, rows_per_gpu, halo_bytes = run_row_sharded(c5, dev, rank, world, 5, 3)
            extra["c5_row_sharded"] = {
                "workload": "c5", "n_gpus": world, "rows_per_gpu": rows_per_gpu, "ms_per_step": tn,
                "ms_per_step_one_gpu_whole_image": t1, "speedup": t1 / tn, "efficiency": t1 / tn / world,
                "halo_bytes_per_step_per_gpu": halo_bytes,
                "value": 3.5 * flops_fwd(*c5[:6]) / (tn * 1e-3) / 1e12, "unit": "TFLOP/s", "scaling": "strong",
                "exchange": "NCCL point-to-point: K/V halo rows received into the extended buffers while the interior "
                            "rows' forward runs; fp32 dK/dV halo partials exchanged while the interior key rows' dK/dV runs"}
    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    kern = {"na2d forward": (ms_fwd, ab["fwd"]), "na2d backward dQ": (ms_dq, ab["dq"]),
            "na2d backward dK/dV": (ms_dkdv, ab["dkdv"])}
    dom = max(kern, key=lambda n: kern[n][0])
    dom_ms, dom_bytes = kern[dom]
    traffic = None
    if args.workload in NCU_DRAM_BYTES and dtype == "bf16" and args.path != "simt":
        traffic = NCU_DRAM_BYTES[args.workload][dom]
    ach = dom_bytes / (dom_ms * 1e-3) / 1e9
    step_ach = ab["step"] / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "effective_tflops_fwd_bwd", "value": flops_step * world / (ms_step * 1e-3) / 1e12,
        "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == "fp32" else dtype, "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "heads": N, "H": H, "W": W, "head_dim": C,
                   "kernel_size": ks, "input_dtype": dtype, "accumulate": "fp32", "path": args.path,
                   "units_per_gpu": B * N, "sharding": "batch x head units, no collective",
                   "l2": "inputs larger than L2" if 8 * ab["T"] + 2 * ab["L"] >= 512 << 20 else "L2 flushed between steps (256 MiB write)"},
        "fwd_ms": ms_fwd, "bwd_dq_ms": ms_dq, "bwd_dkdv_ms": ms_dkdv,
        "fwd_tflops": flops_fwd(*shape, ks) / (ms_fwd * 1e-3) / 1e12,
        "bwd_tflops": 2.5 * flops_fwd(*shape, ks) / ((ms_dq + ms_dkdv) * 1e-3) / 1e12,
        "tensor_roofline_frac": flops_step / (ms_step * 1e-3) / 1e12 / tensor_peak if tensor_peak else None,
        "roofline": {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                     "frac": ach / hbm_peak, "traffic": traffic,
                     "traffic_source": NCU_TRAFFIC_SOURCE if traffic else None, "peak_source": peak_kind,
                     "algorithmic_bytes_per_launch": dom_bytes,
                     "per_kernel_frac": {n: round(b / (ms * 1e-3) / 1e9 / hbm_peak, 4) for n, (ms, b) in kern.items()}},
        "roofline_step": {"bound": "hbm", "achieved": step_ach, "peak": hbm_peak, "unit": "GB/s",
                          "frac": step_ach / hbm_peak, "algorithmic_bytes": ab["step"]},
        "gpu_launches": launches, "clocks": clocks,
    }
    if e2e:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        t_cpu, fl_cpu, what = cpu_port_sample(wl, 12.0, threads)
        line["cpu_baseline"] = {"value": fl_cpu / t_cpu / 1e12, "unit": "TFLOP/s", "cores": threads,
                                "kind": "port", "sample": what, "seconds": t_cpu}
        ref = cpu_reference_sample(WORKLOADS["c1"], 10.0, threads)
        if ref is not None:                             # the reference's own code on its CPU-runnable configuration
            t_ref, fl_ref, what_ref = ref
            line["cpu_baseline"]["reference_c1"] = {
                "value": fl_ref / t_ref / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "reference",
                "sample": what_ref, "seconds": t_ref,
                "note": "its backward fills dQ for the first 3x3 tile only (e_natten/pytorch.py:228-231); nominal flops"}
            t2, f2, w2 = cpu_reference_sample(wl, 10.0, threads)
            line["cpu_baseline"]["reference_sample"] = {"value": f2 / t2 / 1e12, "unit": "TFLOP/s", "cores": threads,
                                                        "kind": "reference", "sample": w2, "seconds": t2}
    if extra:
        line["extra"] = extra
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
