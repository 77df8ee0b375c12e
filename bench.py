"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload quant|linear|train] [--impl reference]

Prints ONE JSON line (rank 0).  Timing: CUDA events on the launching stream, max over ranks, inputs
rotated through a set larger than the 126 MB L2 so no timed step finds its input cached.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "sm120-nvfp4-training_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np
import torch

C1_BYTES_PER_PASS = 4096 * 4096 * 2 + 4096 * 2048 + 4096 * 4096 // 16 + 4  # 42,991,620


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.stop = [], set(), threading.Event()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {}
        for key in ("HwSlowdown", "HwThermalSlowdown", "SwThermalSlowdown", "SwPowerCap", "HwPowerBrakeSlowdown"):
            val = getattr(nv, "nvmlClocksThrottleReason" + key, None)
            if val is not None:
                names[val] = key
        while not self.stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self.stop.wait(0.05)

    def __enter__(self):
        if self.nv is not None:
            self.thread.start()
        return self

    def __exit__(self, *_):
        self.stop.set()
        if self.nv is not None:
            self.thread.join(timeout=2)

    def summary(self):
        snake = {"HwSlowdown": "hw_slowdown", "HwThermalSlowdown": "hw_thermal_slowdown", "SwThermalSlowdown": "sw_thermal_slowdown",
                 "SwPowerCap": "sw_power_cap", "HwPowerBrakeSlowdown": "hw_power_brake"}
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(snake[r] for r in self.reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def max_over_ranks(ms: float, world: int, device) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def c1_input(seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((4096, 4096), generator=g)
    pos = torch.randperm(4096 * 4096, generator=g)[:16777]
    x.view(-1)[pos] *= 50
    return x.bfloat16()


# ------------------------------------------------------------------------------------------------
# workload: quantise + dequantise of 4096 x 4096 BF16 (RNE pass and Philox-SR pass, both with H16 RHT)
# ------------------------------------------------------------------------------------------------
def run_quant(args, rank, world, device):
    import oracle as O
    from nvfp4_training import _native as nat

    nbuf = 8  # 8 x 32 MiB of input = 256 MiB, twice the L2
    base = c1_input(rank)
    host = [base.roll(i, 0).contiguous().pin_memory() for i in range(nbuf)]
    dev = [h.to(device) for h in host]
    signs = torch.from_numpy(O.default_signs(0)).to(device)
    out_bf16 = torch.empty((4096, 4096), dtype=torch.bfloat16, device=device)
    launches = 0

    def step(i, x=None):
        nonlocal launches
        x = dev[i % nbuf] if x is None else x
        p, s, t = nat.quantize(x, signs, 4096, 4096, 0, True, 0)
        nat.dequantize(p, s, t, 4096, 4096, dtype=torch.bfloat16)
        p2, s2, t2 = nat.quantize(x, signs, 4096, 4096, nat.Q_SR_PHILOX, True, 0)
        nat.dequantize(p2, s2, t2, 4096, 4096, dtype=torch.bfloat16)
        launches += 6
        return p2, s2, t2

    for i in range(args.warmup):
        step(i)
    barrier(world)
    launches = 0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch.cuda.current_device()) as clk:
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        barrier(world)
    ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps, world, device)
    timed_launches = launches
    bytes_per_step = 4 * C1_BYTES_PER_PASS
    value = world * bytes_per_step / (ms * 1e-3) / 1e9

    # dominant kernel alone: the tile quantiser with the tensor scale given (RNE + RHT), rotated inputs
    pts = nat.amax(dev[0])[2:3].clone()
    reps = max(20, args.steps)
    for i in range(3):
        nat.quantize(dev[i % nbuf], signs, 4096, 4096, 0, True, 0, given_scale=pts)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for i in range(reps):
        nat.quantize(dev[i % nbuf], signs, 4096, 4096, 0, True, 0, given_scale=pts)
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / reps
    pk = peaks()
    achieved = C1_BYTES_PER_PASS / (kernel_ms * 1e-3) / 1e9

    # end to end through the operator with host buffers: H2D of the input, D2H of payload + scales + pts
    out_p = torch.empty((4096, 2048), dtype=torch.uint8).pin_memory()
    out_s = torch.empty((1024, 1024), dtype=torch.uint8).pin_memory()
    out_t = torch.empty((), dtype=torch.float32).pin_memory()
    staged = torch.empty_like(dev[0])
    def e2e_step(i):
        staged.copy_(host[i % nbuf], non_blocking=True)
        p, s, t = step(i, staged)
        out_p.copy_(p, non_blocking=True); out_s.copy_(s, non_blocking=True); out_t.copy_(t, non_blocking=True)
    for i in range(3):
        e2e_step(i)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        e2e_step(i)
    e1.record()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps, world, device)
    h2d = host[0].numel() * 2
    d2h = out_p.numel() + out_s.numel() + 4

    line = {
        "metric": "nvfp4_quantize_dequantize_GBps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16->e2m1/ue4m3 (fp32 math)", "data": "synthetic",
        "config": {"workload": "C1: 4096x4096 BF16 N(0,1) + 0.1% x50 outliers per GPU; per step RNE+RHT quantise, dequantise, "
                               "Philox-SR+RHT quantise (seed 0), dequantise; sign seed 0", "l2": "8 rotated inputs (256 MiB > L2)",
                   "rows_sharded_across_gpus": world},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "traffic": None, "kernel": "quant_tile_kernel<bf16,row> (RNE+RHT, scale given)", "kernel_ms": kernel_ms,
                     "peak_source": pk["source"]},
        "e2e": {"value": world * bytes_per_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": timed_launches,
        "clocks": clk.summary(),
    }
    if rank == 0 and world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_quant_baseline(base)
    return line


def cpu_quant_baseline(base: torch.Tensor, budget_s: float = 12.0):
    """The oracle on the host cores: same four passes on the same tensor, repeated inside a time budget."""
    import oracle as O
    xo = base.view(torch.int16).numpy().view(np.uint16)
    signs = O.default_signs(0)
    cores = os.cpu_count() or 1
    t0 = time.perf_counter()
    reps = 0
    while True:
        p, s, t = O.quantize(xo, rht=True, signs=signs)
        O.dequantize(p, s, t, 4096, 4096)
        p, s, t = O.quantize(xo, sr_mode=O.SR_PHILOX, rht=True, signs=signs, seed=0)
        O.dequantize(p, s, t, 4096, 4096)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 20:
            break
    return {"value": reps * 4 * C1_BYTES_PER_PASS / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{reps} full C1 steps (4 passes each) on the OpenMP C oracle"}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    base = c1_input(0)
    for _ in range(min(args.warmup, 1)):
        cpu_quant_baseline(base, budget_s=1.0)
    res = cpu_quant_baseline(base, budget_s=max(5.0, 2.0 * args.steps))
    ms = 4 * C1_BYTES_PER_PASS / (res["value"] * 1e9) * 1e3
    return {"impl": "reference", "metric": "nvfp4_quantize_dequantize_GBps", "value": res["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16->e2m1/ue4m3 (fp32 math)", "data": "synthetic",
            "config": {"workload": "C1: 4096x4096 BF16; CPU restatement of the reference kernels (the reference itself needs an SM120 GPU)"},
            "cpu_baseline": res, "e2e": {"value": res["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="quant")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world, local = dist_env()
    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the NVFP4 path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    line = {"quant": run_quant}[args.workload](args, rank, world, device)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
