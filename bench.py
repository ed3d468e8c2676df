#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line (rank 0).  See DESIGN.md for the definition of every field.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
ROTATE_BYTES = 512 * 1024 * 1024          # distinct operand bytes touched per rotation (> 2x L2)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# clocks sampling during the timed region
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self._stop = threading.Event()
        self._thread = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.gpu_index)], capture_output=True, text=True, timeout=5).stdout
                for line in out.strip().splitlines():
                    self.rows.append([c.strip() for c in line.split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            except (ValueError, IndexError):
                continue
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
class Workload:
    """A workload owns R rotating copies of its streamed operands (R * bytes >= ROTATE_BYTES), so
    that every launch in a rotation reads operands that are not in L2."""
    name = ""
    unit_name = ""

    def launches_per_rotation(self):
        raise NotImplementedError


class Q4MatvecC1(Workload):
    """BASELINE config C1: q4 matvec, batch 1, W[4096,4096] group 64, fp16 scale/zero, seed 1001."""
    name = "c1_q4_matvec_b1_4096x4096_g64"
    bits, B, N, K, G, seed = 4, 1, 4096, 4096, 64, 1001

    def __init__(self, pkg, device):
        self.q = importlib.import_module(f"{entry.PKG_ALIAS}.ops.quant_ops")
        synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
        w, s, z = synth.quantized_weight(self.N, self.K, self.bits, self.G, seed=self.seed)
        self.host = (w, s, z)
        self.bytes = w.numel() + s.numel() * 2 + z.numel() * 2 + self.B * self.K * 2 + self.B * self.N * 2
        self.R = max(2, -(-ROTATE_BYTES // self.bytes))
        self.w = [w.to(device).clone() for _ in range(self.R)]
        self.s = [s.to(device).clone() for _ in range(self.R)]
        self.z = [z.to(device).clone() for _ in range(self.R)]
        self.x_host = synth.activations((self.B, self.K), self.seed + 500).pin_memory()
        self.x = self.x_host.to(device)
        self.device = device

    def algorithmic_bytes(self):
        return self.bytes

    def rotation(self):
        """One pass over all R copies; returns the last output."""
        y = None
        fn = self.q.q4_matvec_decode if self.bits == 4 else self.q.q8_matvec_decode
        for i in range(self.R):
            y = fn(self.x, self.w[i], self.s[i], self.z[i], group_size=self.G, backend="cuda")
        return y

    def launches_per_rotation(self):
        return self.R

    def e2e_call(self, i):
        """Public API with host buffers: H2D of the activation row, matvec, D2H of the result."""
        fn = self.q.q4_matvec_decode if self.bits == 4 else self.q.q8_matvec_decode
        x = self.x_host.to(self.device, non_blocking=True)
        y = fn(x, self.w[i % self.R], self.s[i % self.R], self.z[i % self.R], group_size=self.G, backend="cuda")
        return y.cpu()

    def e2e_bytes(self):
        return self.B * self.K * 2, self.B * self.N * 2

    def cpu_reference_call(self):
        from oracle import quant_ops as oq
        w, s, z = self.host
        fn = oq.reference_q4_matvec_decode if self.bits == 4 else oq.reference_q8_matvec_decode
        return fn(self.x_host, w, s, z, group_size=self.G)


WORKLOADS = {"c1": Q4MatvecC1}


# ------------------------------------------------------------------------------------------------
def time_graph(workload, steps, warmup, stream):
    """Captures one rotation in a CUDA graph and replays it; returns seconds per step (rotation)."""
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        workload.rotation()                      # lazy init outside capture (function attributes, caches)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            workload.rotation()
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(steps):
            graph.replay()
        end.record(stream)
        end.synchronize()
    return start.elapsed_time(end) / 1e3 / steps


def run_own(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    pkg = entry.load_package()
    cabi = importlib.import_module(f"{entry.PKG_ALIAS}.ops._cabi")
    cabi.load()
    wl = WORKLOADS[args.workload](pkg, device)
    stream = torch.cuda.Stream(device)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    barrier()
    with ClockSampler(local) as clocks:
        sec_per_step = time_graph(wl, args.steps, max(3, args.warmup), stream)
    barrier()
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([sec_per_step], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sec_per_step = float(t.item())
    launches = wl.launches_per_rotation()
    sec_per_launch = sec_per_step / launches
    peak, peak_kind = measured_peaks()
    achieved = wl.algorithmic_bytes() / sec_per_launch / 1e9

    # end to end through the public API with host buffers
    n_e2e = max(20, min(200, args.steps * 4))
    for i in range(5):
        wl.e2e_call(i)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n_e2e):
        wl.e2e_call(i)
    torch.cuda.synchronize()
    e2e_sec = (time.perf_counter() - t0) / n_e2e
    h2d, d2h = wl.e2e_bytes()

    status = cabi.device_status()
    line = {
        "metric": "q4 matvec achieved HBM bandwidth (algorithmic bytes / kernel time)",
        "value": round(achieved * world, 2),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(3, args.warmup),
        "ms_per_step": round(sec_per_step * 1e3, 5),
        "us_per_launch": round(sec_per_launch * 1e6, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16 activations, u4 codes, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": wl.name, "cache": f"cold: {wl.R} rotating operand copies = {wl.R * wl.algorithmic_bytes() >> 20} MiB > L2",
                   "launches_per_step": launches},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": None, "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": wl.algorithmic_bytes()},
        "e2e": {"value": round(wl.algorithmic_bytes() / e2e_sec / 1e9 * world, 3), "unit": "GB/s",
                "us_per_call": round(e2e_sec * 1e6, 2), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * args.steps,
        "clocks": clocks.summary(),
        "device_status": status,
    }
    if rank == 0:
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(wl, budget_s=10.0)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def cpu_baseline(wl, budget_s):
    torch.set_num_threads(os.cpu_count() or 1)
    wl.cpu_reference_call()
    n, t0 = 0, time.perf_counter()
    while n < 3 or (time.perf_counter() - t0 < budget_s and n < 50):
        wl.cpu_reference_call()
        n += 1
    sec = (time.perf_counter() - t0) / n
    return {"value": round(wl.algorithmic_bytes() / sec / 1e9, 4), "unit": "GB/s", "us_per_call": round(sec * 1e6, 1),
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n} calls of the torch-CPU restatement of the reference path (dequantise W to fp16, fp32 matmul) on {wl.name}"}


class _HostOnly:
    """Workload inputs for the reference arm without touching a GPU."""


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    entry.load_package()
    synth = importlib.import_module(f"{entry.PKG_ALIAS}.synth")
    cls = WORKLOADS[args.workload]
    wl = _HostOnly()
    wl.__class__ = type("HostWorkload", (cls,), {"__init__": lambda self: None})
    w, s, z = synth.quantized_weight(cls.N, cls.K, cls.bits, cls.G, seed=cls.seed)
    wl.host = (w, s, z)
    wl.x_host = synth.activations((cls.B, cls.K), cls.seed + 500)
    wl.bytes = w.numel() + s.numel() * 2 + z.numel() * 2 + cls.B * cls.K * 2 + cls.B * cls.N * 2
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(max(3, args.warmup)):
        wl.cpu_reference_call()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.cpu_reference_call()
    sec = (time.perf_counter() - t0) / args.steps
    value = round(wl.bytes / sec / 1e9, 4)
    line = {
        "impl": "reference",
        "metric": "q4 matvec achieved HBM bandwidth (algorithmic bytes / kernel time)",
        "value": value, "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": round(sec * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 activations, u4 codes, f32 accumulate", "data": "synthetic",
        "config": {"workload": cls.name},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"each step = one call of the torch-CPU restatement of the reference path on {cls.name}"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--workload", default="c1", choices=sorted(WORKLOADS))
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_own(args)


if __name__ == "__main__":
    main()
