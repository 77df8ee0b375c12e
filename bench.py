"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload train|quant] [--impl reference]

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


class ProfilerRange:
    """cudaProfilerStart/Stop around the timed region (--profiler-range), so that a profiler started with
    --profile-from-start off sees exactly the timed launches."""

    def __init__(self, enabled: bool):
        self.enabled = enabled

    def __enter__(self):
        if self.enabled:
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
        return self

    def __exit__(self, *_):
        if self.enabled:
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()


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
    from nvfp4_training import _native as nat
    from nvfp4_training._backend.quant import get_signs

    nbuf = 8  # 8 x 32 MiB of input = 256 MiB, twice the L2
    base = c1_input(rank)
    host = [base.roll(i, 0).contiguous().pin_memory() for i in range(nbuf)]
    dev = [h.to(device) for h in host]
    signs = get_signs(device, seed=0)     # this benchmark configuration names sign seed 0; the package default is 1
    out_bf16 = torch.empty((4096, 4096), dtype=torch.bfloat16, device=device)
    # a 4096 x 4096 BF16 tensor fits shared memory: the operator takes amax, scale and packing in one cooperative launch
    # (two launches, amax then quantiser, with NVFP4_QUANT_RESIDENT=0)
    per_step = 4 if os.environ.get("NVFP4_QUANT_RESIDENT", "1") != "0" else 6

    def step(i, x=None):
        x = dev[i % nbuf] if x is None else x
        p, s, t = nat.quantize(x, signs, 4096, 4096, 0, True, 0)
        nat.dequantize(p, s, t, 4096, 4096, dtype=torch.bfloat16)
        p2, s2, t2 = nat.quantize(x, signs, 4096, 4096, nat.Q_SR_PHILOX, True, 0)
        nat.dequantize(p2, s2, t2, 4096, 4096, dtype=torch.bfloat16)
        return p2, s2, t2

    for i in range(args.warmup):
        step(i)
    barrier(world)
    clk = ClockSampler(torch.cuda.current_device())
    ms, _ = graph_time(step, args.steps, device, args.profiler_range, clk)   # the K timed steps are one graph replay
    barrier(world)
    ms = max_over_ranks(ms, world, device)
    timed_launches = per_step * args.steps
    bytes_per_step = 4 * C1_BYTES_PER_PASS
    value = world * bytes_per_step / (ms * 1e-3) / 1e9

    # dominant kernel alone: the tile quantiser with the tensor scale given (RNE + RHT), rotated inputs
    pts = nat.amax(dev[0])[2:3].clone()
    reps = max(24, args.steps)
    kernel_ms, _ = graph_time(lambda i: nat.quantize(dev[i % nbuf], signs, 4096, 4096, 0, True, 0, given_scale=pts), reps, device)
    amax_ms, _ = graph_time(lambda i: nat.amax(dev[i % nbuf]), reps, device)
    op_ms, _ = graph_time(lambda i: nat.quantize(dev[i % nbuf], signs, 4096, 4096, 0, True, 0), reps, device)   # amax included
    sr_ms, _ = graph_time(lambda i: nat.quantize(dev[i % nbuf], signs, 4096, 4096, nat.Q_SR_PHILOX, True, 0, given_scale=pts), reps, device)
    deq_in = nat.quantize(dev[0], signs, 4096, 4096, 0, True, 0)
    deq_ms, _ = graph_time(lambda i: nat.dequantize(deq_in[0], deq_in[1], deq_in[2], 4096, 4096, dtype=torch.bfloat16), reps, device)
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
                               "Philox-SR+RHT quantise (seed 0), dequantise; sign seed 0", "l2": "8 rotated inputs (256 MiB > L2)", "timing": "the timed steps are captured once and replayed as one CUDA graph",
                   "rows_sharded_across_gpus": world},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "traffic": NCU_TRAFFIC["quant_c1"], "traffic_source": NCU_TRAFFIC_SOURCE["quant_c1"],
                     "kernel": "quant_stream_kernel<bf16,row,RNE,RHT> (scale given)", "timing": "30 launches on rotated inputs captured as one CUDA graph, CUDA events around the replay", "kernel_ms": kernel_ms,
                     "peak_source": pk["source"]},
        "e2e": {"value": world * bytes_per_step / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "kernels_us": {"amax": amax_ms * 1e3, "quantize_rne_rht": kernel_ms * 1e3, "quantize_philox_sr_rht": sr_ms * 1e3,
                       "dequantize_bf16": deq_ms * 1e3, "operator_rne_rht_amax_included": op_ms * 1e3},
        "operator_frac_of_hbm": C1_BYTES_PER_PASS / (op_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
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


# ------------------------------------------------------------------------------------------------
# workload: packed NVFP4 linear layer, forward + dgrad + wgrad (config 2) -- GEMM TFLOP/s
# ------------------------------------------------------------------------------------------------
C2 = dict(tokens=8192, d_in=4096, d_out=4096)
FP4_NOMINAL_TFLOPS = 9000.0
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch from the ncu captures summarised under profiles/
# (one capture per kernel; outputs still resident in the 126 MB L2 at kernel end are not in them)
NCU_TRAFFIC = {"gemm_c2": (50.2e6 + 50.6e6 + 42.3e6) / 3, "quant_c1": 33.6e6, "adamw": 287.1e6}
NCU_TRAFFIC_SOURCE = {"gemm_c2": "profiles/gemm_kernel_c2.md", "quant_c1": "profiles/quant_stream_kernel_c1.md",
                      "adamw": "profiles/adamw_kernel_balanced.md"}


def graph_time(fn, n, device, profiler_range=False, clock=None):
    """Device time per call of fn(i), i = 0..n-1, with the n calls captured once as a CUDA graph and replayed: kernels of a
    few tens of microseconds would otherwise be timed at the host's launch rate.  Returns (ms per call, last result)."""
    from nvfp4_training import _native as nat
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        nat.scratch(device)            # the stream's scratch block exists before capture
        for i in range(min(n, 3)):
            fn(i)
        torch.cuda.synchronize(device)
        with torch.cuda.graph(graph, stream=side):
            out = None
            for i in range(n):
                out = fn(i)
    torch.cuda.synchronize(device)
    graph.replay()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ProfilerRange(profiler_range):
        if clock is not None:
            clock.__enter__()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize(device)
        if clock is not None:
            clock.__exit__(None, None, None)
    return e0.elapsed_time(e1) / n, out


def time_kernel(fn, reps, profiler_range=False):
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ProfilerRange(profiler_range):
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def gemm_microbench(device, tokens, d_in, d_out, reps=20, profiler_range=False):
    """The three GEMMs of one layer on rotated operand sets; returns (ms per triple, TFLOP/s, launches)."""
    from nvfp4_training._backend import quant
    g = torch.Generator(device=device).manual_seed(1234)
    sets = []
    for _ in range(3):   # 3 operand sets x ~150 MB > L2
        x = torch.randn((tokens, d_in), device=device, generator=g).bfloat16()
        w = torch.randn((d_out, d_in), device=device, generator=g) * 0.02
        gy = (torch.randn((tokens, d_out), device=device, generator=g) * 1e-3).bfloat16()
        signs = quant.get_signs(device)
        a, xt = quant.dual(x, signs)
        wd, ws, wp, wtd, wts = quant.pair(w, quant.weight_scale(w))
        ga, gt = quant.dual(gy, signs, sr=True, offset=1234)
        sets.append((a, xt, quant.Packed(wd, ws, wp, torch.bfloat16), quant.Packed(wtd, wts, wp, torch.bfloat16), ga, gt))

    def triple(i):
        a, xt, w, wt, ga, gt = sets[i % len(sets)]
        quant.matmul(a, w, rows=tokens, cols=d_out, output_dtype=torch.bfloat16)
        quant.matmul(ga, wt, rows=tokens, cols=d_in, output_dtype=torch.bfloat16)
        quant.raw_matmul(gt, xt, d_out, d_in)
    ms = time_kernel(triple, reps, profiler_range)
    flops = 3 * 2.0 * tokens * d_in * d_out
    return ms, flops / (ms * 1e-3) / 1e12


def quant_microbench(device, reps=30):
    """The quantise operator with amax included (one cooperative launch at this size) on rotated 4096x4096 BF16 inputs,
    RNE + RHT: GB/s over the single-read bytes."""
    from nvfp4_training._backend import quant
    xs = [c1_input(i).to(device) for i in range(8)]
    signs = quant.get_signs(device)
    ms, _ = graph_time(lambda i: quant.quantize(xs[i % 8], rht=True, signs=signs), reps, device)
    return ms, C1_BYTES_PER_PASS / (ms * 1e-3) / 1e9


# ------------------------------------------------------------------------------------------------
# workload: full-parameter training step of the ~3.8B decoder (config 3), data parallel over the ranks
# ------------------------------------------------------------------------------------------------
C3 = dict(layers=32, dim=3072, heads=24, ffn=8192, vocab=32000, seq=2048, micro_batch=4)


def build_c3(cfg, world, device):
    import nvfp4_training as nv
    from nvfp4_training._workloads.llama import Decoder
    torch.manual_seed(0)
    with torch.device(device):
        model = Decoder(layers=cfg["layers"], dim=cfg["dim"], heads=cfg["heads"], ffn=cfg["ffn"], vocab=cfg["vocab"], seq=cfg["seq"])
    model = nv.enable_nvfp4(model, profile="balanced", lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    model.nvfp4_optimizer.param_groups[0]["prepack"] = os.environ.get("NVFP4_PREPACK", "0") == "1"
    if world > 1:
        nv.enable_data_parallel(model, depth=int(os.environ.get("NVFP4_DP_DEPTH", "2")))
    return model


def time_c3(model, cfg, ids, steps, warmup, world, device, profiler_range=False, e2e=True):
    """Capture the whole step once, replay it: (ms per step device-timed, ms per step with host inputs, losses, calls, clocks)."""
    import nvfp4_training as nv
    from nvfp4_training._workloads.llama import token_loss
    x0, y0 = ids[0, :, :-1].to(device), ids[0, :, 1:].to(device)
    total = warmup + 2 * steps + 2
    graph = nv.capture_step(model, token_loss, x0, y0, steps=total)
    calls = graph.library_calls
    dev_ids = ids.to(device)
    losses, e2e_ms = [], None
    with graph:
        i = 0
        for _ in range(warmup):
            graph.step(dev_ids[i, :, :-1], dev_ids[i, :, 1:]); i += 1
        barrier(world)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(torch.cuda.current_device()) as clk, ProfilerRange(profiler_range):
            ev0.record()
            for _ in range(steps):
                loss = graph.step(dev_ids[i, :, :-1], dev_ids[i, :, 1:]); i += 1
            ev1.record()
            barrier(world)
        ms = max_over_ranks(ev0.elapsed_time(ev1) / steps, world, device)
        losses.append(float(loss.item()))
        if e2e:
            # end to end: token ids come from pinned host memory, the loss goes back to the host, every step
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            xb, yb = torch.empty_like(x0), torch.empty_like(y0)
            barrier(world)
            e0.record()
            for _ in range(steps):
                xb.copy_(ids[i, :, :-1], non_blocking=True); yb.copy_(ids[i, :, 1:], non_blocking=True)
                losses.append(float(graph.step(xb, yb).item())); i += 1
            e1.record()
            barrier(world)
            e2e_ms = max_over_ranks(e0.elapsed_time(e1) / steps, world, device)
    return ms, e2e_ms, losses, calls, clk.summary()


def incumbent_gemm_tflops(device, tokens, d_in, d_out, reps=20):
    """The library's NVFP4 GEMM (torch._scaled_mm -> cuBLASLt) on the same packed operands, for comparison only; None when
    this torch build does not accept them."""
    try:
        from nvfp4_training._backend import quant
        f4, f8 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
        x = torch.randn((tokens, d_in), device=device).bfloat16()
        w = (torch.randn((d_out, d_in), device=device) * 0.02).bfloat16()
        a, b = quant.quantize(x), quant.quantize(w)
        run = lambda i: torch._scaled_mm(a.data.view(f4), b.data.view(f4).t(), a.scale.view(f8), b.scale.view(f8), out_dtype=torch.bfloat16)
        ms = time_kernel(run, reps)
        return 2.0 * tokens * d_in * d_out / (ms * 1e-3) / 1e12
    except Exception:
        return None


def run_train(args, rank, world, device):
    import nvfp4_training as nv
    from nvfp4_training import _native as nat
    from nvfp4_training._workloads.llama import linear_parameters, warm_attention
    os.environ.setdefault("NVFP4_SR_RNG", "philox")
    sr_rng = os.environ["NVFP4_SR_RNG"].lower()
    cfg = dict(C3)
    if args.layers:
        cfg["layers"] = args.layers
    mb, seq = cfg["micro_batch"], cfg["seq"]
    tokens = mb * seq
    total = args.warmup + 2 * args.steps + 2
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg["vocab"], (total, world, mb, seq + 1), generator=gen)[:, rank].contiguous().pin_memory()
    model = build_c3(cfg, world, device)
    n_linear = linear_parameters(model)
    n_params = sum(p.numel() for p in model.parameters())
    warm_attention(model, mb, seq, device)
    torch.cuda.reset_peak_memory_stats()
    ms, e2e_ms, losses, captured_calls, clocks = time_c3(model, cfg, ids, args.steps, args.warmup, world, device, args.profiler_range)
    nv.check_finite(model)
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30
    comm = None
    if world > 1:
        # the same captured step with the collectives left out (timing only): what the gradient exchange costs the step
        red = model.nvfp4_optimizer.reducer
        per_step = dict(collectives=red.collectives, bytes=sum(p.numel() * (2 if red.has_slot(p) else 4) for p in model.parameters()))
        red.elide = True
        quiet_ms = time_c3(model, cfg, ids, max(3, args.steps // 2), 3, world, device, e2e=False)[0]
        red.elide = False
        comm = {"ms_per_step_with_collectives": ms, "ms_per_step_collectives_elided": quiet_ms, "exposed_ms": ms - quiet_ms,
                "collectives_per_step": per_step["collectives"], "bytes_reduced_per_step": per_step["bytes"],
                "note": "elided = the same graph captured without the all-reduces; results of that run are discarded"}
    variants = {}
    if world == 1 and not args.no_variants:
        # the same step with the reference's integer-hash stochastic rounding (bit-exact to the reference's generator)
        del model
        torch.cuda.empty_cache()
        other = "hash" if sr_rng == "philox" else "philox"
        os.environ["NVFP4_SR_RNG"] = other
        alt = build_c3(cfg, world, device)
        alt_ms = time_c3(alt, cfg, ids, max(3, args.steps // 2), 3, world, device, e2e=False)[0]
        os.environ["NVFP4_SR_RNG"] = sr_rng
        variants[f"sr_rng_{other}"] = {"ms_per_step": alt_ms, "tokens_per_s": tokens / (alt_ms * 1e-3)}
        del alt
        torch.cuda.empty_cache()
    pk = peaks()
    gemm_ms, gemm_tf = gemm_microbench(device, tokens, cfg["dim"], cfg["ffn"])
    c2_ms, c2_tf = gemm_microbench(device, C2["tokens"], C2["d_in"], C2["d_out"])
    q_ms, q_gbs = quant_microbench(device)
    fp4_peak = 4.0 * pk["bf16_tflops"]
    linear_flops = 6.0 * n_linear * tokens
    # lower bound of the step from its three kinds of work: FP4 GEMMs at the tensor peak, BF16 attention at the sustained
    # BF16 peak, optimizer and quantiser traffic at the HBM peak
    attn_flops = 3.5 * cfg["layers"] * 4.0 * mb * seq * seq * cfg["dim"] / 2
    adam_bytes = 10.0 * n_params
    quant_bytes = 3.125 * (2 * n_linear + tokens * cfg["layers"] * 2 * (cfg["dim"] * 3 + cfg["ffn"]) + tokens * cfg["layers"] * (4 * cfg["dim"] + 2 * cfg["ffn"]))
    bound_ms = (linear_flops / (fp4_peak * 1e12) + attn_flops / ((pk["bf16_sustained"] or pk["bf16_tflops"]) * 1e12)
                + (adam_bytes + quant_bytes) / (pk["hbm_gbs"] * 1e9)) * 1e3
    line = {
        "metric": "nvfp4_train_tokens_per_s", "value": world * tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 x ue4m3 block scales, fp32 accumulate); bf16 attention", "data": "synthetic",
        "config": {"workload": f"C3: Llama-style decoder {n_params / 1e9:.2f}B params ({cfg['layers']} layers, d {cfg['dim']}, {cfg['heads']} heads, "
                               f"SwiGLU {cfg['ffn']}, vocab {cfg['vocab']}; q/k/v and gate/up as fused projections), seq {seq}, micro-batch {mb} "
                               "per GPU, balanced profile, compressed AdamW lr 3e-4 betas (0.9,0.95) wd 0.1, whole step replayed as one CUDA graph",
                   "global_batch": world * mb, "seq_len": seq, "parallelism": f"dp{world}",
                   "sr_rng": {"philox": "philox4x32-10 bits into the hardware stochastic conversion (cvt.rs.e2m1x4)",
                              "hash": "the reference's 32-bit integer hash, 24-bit uniforms"}[sr_rng],
                   "prepack": os.environ.get("NVFP4_PREPACK", "0") == "1",
                   "l2": "per-step working set (weights 7.6 GB + activations) exceeds the 126 MB L2"},
        "tokens_per_s_per_gpu": tokens / (ms * 1e-3), "train_peak_GiB": peak_gib, "loss": losses[0],
        "linear_tflops_in_step": linear_flops / (ms * 1e-3) / 1e12,
        "roofline": {"bound": "tensor", "achieved": gemm_tf, "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tf / fp4_peak,
                     "traffic": NCU_TRAFFIC["gemm_c2"] * (tokens * cfg["dim"] + cfg["dim"] * cfg["ffn"] + tokens * cfg["ffn"])
                     / (C2["tokens"] * C2["d_in"] + C2["d_in"] * C2["d_out"] + C2["tokens"] * C2["d_out"]),
                     "traffic_source": NCU_TRAFFIC_SOURCE["gemm_c2"] + ", per launch, scaled to this layer by the sum of the three matrices' sizes",
                     "kernel": f"gemm_kernel<256, paired CTAs> fprop+dgrad+wgrad of a {cfg['dim']}x{cfg['ffn']} layer at {tokens} tokens",
                     "kernel_ms": gemm_ms, "timing": "CUDA events around 20 eager launches of the triple on rotated operand sets, after the timed "
                     "training region (87 us per launch, far above the host's launch interval)",
                     "peak_source": pk["source"] + " bf16 GEMM x4 (FP4 issue rate)", "frac_of_nominal_9PF": gemm_tf / FP4_NOMINAL_TFLOPS,
                     "step_bound_ms": bound_ms, "step_frac": bound_ms / ms},
        "kernels": {"c2_linear_gemm_tflops": c2_tf, "c2_ms": c2_ms, "c1_quantize_GBps": q_gbs, "c1_quantize_ms": q_ms,
                    "c1_frac_of_hbm": q_gbs / pk["hbm_gbs"],
                    "incumbent_c2_fprop_tflops": incumbent_gemm_tflops(device, C2["tokens"], C2["d_in"], C2["d_out"])},
        "e2e": {"value": world * tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": int(2 * mb * seq) * 8,
                "d2h_bytes_per_step": 4, "steps": args.steps},
        "gpu_launches": captured_calls * args.steps,
        "clocks": clocks,
    }
    if variants:
        line["variants"] = variants
    if comm:
        line["comm"] = comm
    if rank == 0 and world == 1 and not args.skip_cpu:
        line["cpu_baseline"] = cpu_train_baseline(cfg)
    return line


CPU_BUDGET_TOKENS = 256   # tokens of the bounded CPU sample, the same in the GPU arm's cpu_baseline and in --impl reference


def cpu_layer_seconds(cfg, budget_tokens):
    """One decoder layer on the oracle: its four NVFP4 linears (fused q/k/v, o, fused gate/up, down) forward + input
    gradient + weight gradient at `budget_tokens` tokens, and the compressed AdamW of those weights."""
    import oracle as O
    d, f = cfg["dim"], cfg["ffn"]
    shapes = [(d, 3 * d), (d, d), (d, 2 * f), (f, d)]
    g = torch.Generator().manual_seed(0)
    t_lin = t_adam = 0.0
    signs = O.default_signs()
    for k, n in shapes:
        x = torch.randn((budget_tokens, k), generator=g).bfloat16()
        gy = (torch.randn((budget_tokens, n), generator=g) * 1e-3).bfloat16()
        w = (torch.randn((n, k), generator=g) * 0.02).half()
        xb, gb, wb = (t.view(torch.int16).numpy().view(np.uint16) for t in (x, gy, w))
        t0 = time.perf_counter()
        row, col = O.dual(xb, signs=signs)
        wr, wc = O.weight_pair(wb, kind="f16")
        O.matmul_packed(row, wr, budget_tokens, n)
        grow, gcol = O.dual(gb, sr_mode=O.SR_HASH, signs=signs, seed=7)
        O.matmul_packed(grow, wc, budget_tokens, k)
        raw = O.matmul_packed(gcol, col, n, k, out_bf16=True)
        t_lin += time.perf_counter() - t0
        m = np.zeros(n * k, np.int8); v = np.zeros(n * k, np.uint8)
        ms, vs = np.zeros(-(-n * k // 512), np.float32), np.zeros(-(-n * k // 512), np.float32)
        grad = O.to_bf16_bits(raw.reshape(-1))
        t0 = time.perf_counter()
        O.adam_update("half16_v8", wb.reshape(-1).copy(), grad, m, v, ms, vs, step=1, key=1, hyper=O.adam_hyper(3e-4, (0.9, 0.95), 1e-8, 0.1, 1), grad_kind=1)
        t_adam += time.perf_counter() - t0
    return t_lin, t_adam


def use_all_host_cores():
    """Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU legs are meant to use every core.  The oracle links the
    system's OpenMP runtime, which torch.set_num_threads does not reach, so that runtime is told directly as well."""
    import ctypes
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass
    return n


def cpu_train_baseline(cfg, budget_tokens=CPU_BUDGET_TOKENS, samples=3):
    """The oracle on the host cores, median of `samples` runs of one layer, extrapolated to the full token count and layer
    count.  Attention, norms, embedding and head are not included: an optimistic CPU figure."""
    use_all_host_cores()
    tokens_full = cfg["micro_batch"] * cfg["seq"]
    runs = sorted(cpu_layer_seconds(cfg, budget_tokens) for _ in range(samples))
    t_lin, t_adam = runs[len(runs) // 2]
    step_s = (t_lin * (tokens_full / budget_tokens) + t_adam) * cfg["layers"]
    return {"value": tokens_full / step_s, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"median of {samples}: one decoder layer's 4 fused linears fwd+dgrad+wgrad at {budget_tokens} tokens ({t_lin:.1f} s) + its "
                      f"compressed AdamW ({t_adam:.1f} s) on the CPU oracle; extrapolated x{tokens_full // budget_tokens} tokens "
                      f"x{cfg['layers']} layers; attention / embedding / head excluded"}


# ------------------------------------------------------------------------------------------------
# kernel workloads: the three GEMMs of one layer (config 2) and the compressed AdamW kernel alone
# ------------------------------------------------------------------------------------------------
def run_gemm(args, rank, world, device):
    """C2: X[8192,4096] BF16, W[4096,4096] FP32, G[8192,4096] BF16; fprop + dgrad + wgrad on packed operands."""
    from nvfp4_training import _native as nat
    t, k, n = C2["tokens"], C2["d_in"], C2["d_out"]
    barrier(world)
    with ClockSampler(torch.cuda.current_device()) as clk:
        ms, tf = gemm_microbench(device, t, k, n, reps=args.steps, profiler_range=args.profiler_range)
    ms = max_over_ranks(ms, world, device)
    nat.check_status()
    pk = peaks()
    fp4_peak = 4.0 * pk["bf16_tflops"]
    flops = 3 * 2.0 * t * k * n
    tf = flops / (ms * 1e-3) / 1e12
    return {"metric": "nvfp4_linear_gemm_tflops", "value": world * tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e2m1 x ue4m3 block scales, fp32 accumulate, bf16 out", "data": "synthetic",
            "config": {"workload": "C2: fprop, dgrad, wgrad GEMMs of a 4096x4096 layer at 8192 tokens per GPU on pre-quantised operands "
                                   "(token rows sharded across GPUs, no collective)", "l2": "3 rotated operand sets (~450 MB > L2)"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": fp4_peak, "unit": "TFLOP/s", "frac": tf / fp4_peak,
                         "traffic": NCU_TRAFFIC["gemm_c2"], "traffic_source": NCU_TRAFFIC_SOURCE["gemm_c2"],
                         "kernel": "gemm_kernel<256, paired CTAs>", "kernel_ms": ms / 3, "peak_source": pk["source"] + " bf16 GEMM x4 (FP4 issue rate)",
                         "frac_of_nominal_9PF": tf / FP4_NOMINAL_TFLOPS},
            "gpu_launches": 3 * args.steps, "clocks": clk.summary()}


ADAM_N = 4096 * 8192   # one 4096x8192 weight: 33.5 M elements, 335 MB of traffic per launch


def run_adamw(args, rank, world, device):
    """The balanced profile's update kernel (FP16 master with SR, int8 m, uint8 sqrt-v, per-512 scales) on rotated tensors."""
    from nvfp4_training import _native as nat
    import math
    n = ADAM_N
    lr, b1, b2, wd = 3e-4, 0.9, 0.95, 0.1

    def hyper(t):
        return dict(lr=lr, decay=1 - lr * wd, b1=b1, b2=b2, c1=1 / (1 - b1 ** t), c2=1 / math.sqrt(1 - b2 ** t), eps=1e-8)
    sets = []
    for i in range(3):
        g = torch.Generator(device=device).manual_seed(i)
        w = (torch.randn(n, device=device, generator=g) * 0.02).half()
        grad = (torch.randn(n, device=device, generator=g) * 1e-3).bfloat16()
        sets.append(dict(p=w, grad=grad, m=torch.zeros(n, dtype=torch.int8, device=device), v=torch.zeros(n, dtype=torch.uint8, device=device),
                         ms=torch.zeros(n // 512, device=device), vs=torch.zeros(n // 512, device=device),
                         scale=torch.empty((), device=device)))
    count = [0]

    def opt_step(i):
        count[0] += 1
        t = count[0]
        s = sets[i % 3]
        nat.adamw_step(s["p"], 17, s["grad"], s["m"], s["v"], s["ms"], s["vs"], vbits=8, mbits=8, nonlinear_m=False, state_block=512,
                       hyper=hyper(t), step=t, key=12345, grad_kind=1, scale_out=s["scale"])
    for i in range(max(args.warmup, 3)):
        opt_step(i)
    barrier(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch.cuda.current_device()) as clk, ProfilerRange(args.profiler_range):
        ev0.record()
        for i in range(args.steps):
            opt_step(i)
        ev1.record()
        barrier(world)
    ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps, world, device)
    pk = peaks()
    bytes_per = ADAM_N * (2 + 2 + 1 + 1 + 2 + 1 + 1) + ADAM_N // 512 * 16   # p, g, m, v in; p, m, v out; scales
    gbs = bytes_per / (ms * 1e-3) / 1e9
    return {"metric": "nvfp4_adamw_GBps", "value": world * gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 math on fp16/int8/uint8 state",
            "data": "synthetic",
            "config": {"workload": "compressed AdamW (balanced: half16_v8) on one 4096x8192 weight per GPU, BF16 gradient",
                       "l2": "3 rotated parameter sets (1 GB > L2)"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "traffic": NCU_TRAFFIC["adamw"], "traffic_source": NCU_TRAFFIC_SOURCE["adamw"],
                         "kernel": "adamw_kernel<17,8,false,false,512>", "kernel_ms": ms, "peak_source": pk["source"]},
            "elements_per_s": ADAM_N / (ms * 1e-3), "gpu_launches": args.steps, "clocks": clk.summary()}


# ------------------------------------------------------------------------------------------------
# LoRA workloads: config 4 (GPT-2-small layout, bases re-packed to NVFP4) and config 5 (DiT trunk over packed checkpoints)
# ------------------------------------------------------------------------------------------------
def run_lora(args, rank, world, device):
    from precision_lora import prepare_lora, capture_lora_step, lora_parameters
    from nvfp4_training._workloads import lora_models as lm
    packed = args.workload == "lora_packed"
    torch.manual_seed(11 if packed else 7)
    if packed:
        blocks = args.blocks or 24
        model = lm.DiT(blocks=blocks, backward_mode=args.backward_mode, device=device, seed=11)
        model, opt = prepare_lora(model, mode="packed_nvfp4", rank=16, alpha=16, target_modules=lm.DIT_TARGETS, lr=1e-4)
        tokens, n_text, dim = 4608, 512, 3072
        gen = torch.Generator(device=device).manual_seed(11 + rank)
        batches = [tuple(torch.randn(shape, device=device, generator=gen).bfloat16() for shape in ((1, tokens - n_text, dim), (1, n_text, dim)))
                   + (torch.randn((1, tokens - n_text, dim), device=device, generator=gen),) for _ in range(2)]
        loss_fn = lm.denoise_loss
        base_params = blocks * (3 * dim * dim + dim * dim + 2 * 12288 * dim)
        name = (f"C5: {blocks}-block DiT trunk (d 3072, 24 heads, GELU FFN 12288) over packed NVFP4 checkpoints, 4096 image + 512 text "
                f"tokens, LoRA r16 on qkv/out/up/down, batch 1, mode packed_nvfp4, backward {args.backward_mode}, eager")
    else:
        blocks = args.blocks or 12
        model = lm.GPT2Small(layers=blocks).to(device).bfloat16()
        model, opt = prepare_lora(model, mode="nvfp4", rank=16, alpha=16, target_modules=lm.GPT2_TARGETS, lr=2e-4)
        tokens = 16 * 1024
        gen = torch.Generator().manual_seed(7 + rank)
        ids = torch.randint(0, 50257, (2, 16, 1025), generator=gen).to(device)
        batches = [(ids[i, :, :-1].contiguous(), ids[i, :, 1:].contiguous()) for i in range(2)]
        loss_fn = lm.lm_loss
        base_params = blocks * (3 * 768 * 768 + 768 * 768 + 2 * 3072 * 768)
        name = (f"C4: GPT-2-small layout ({blocks} blocks, d 768, vocab 50257), bases re-packed to NVFP4 with RHT, LoRA r16 on "
                "qkv/proj/up/down, 16 x 1024 tokens, mode nvfp4, update captured as one CUDA graph")
    torch.cuda.reset_peak_memory_stats()

    def eager(i):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = loss_fn(model, *batches[i % 2])
        loss.backward()
        opt.step()
        return loss
    graph = None
    if not packed:
        graph = capture_lora_step(model, opt, loss_fn, *batches[0])
    run = (lambda i: graph.step(*batches[i % 2])) if graph is not None else eager
    for i in range(args.warmup):
        run(i)
    barrier(world)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(torch.cuda.current_device()) as clk, ProfilerRange(args.profiler_range):
        ev0.record()
        for i in range(args.steps):
            loss = run(i)
        ev1.record()
        barrier(world)
    ms = max_over_ranks(ev0.elapsed_time(ev1) / args.steps, world, device)
    final = float(loss.item())
    if graph is not None:
        graph.close()
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30
    base_flops = 4.0 * base_params * tokens   # forward + input gradient of the frozen bases
    return {"metric": "lora_tokens_per_s", "value": world * tokens / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "nvfp4 bases (fp32 accumulate), bf16 adapters / attention", "data": "synthetic",
            "config": {"workload": name, "l2": "frozen bases exceed the 126 MB L2" if packed else "activations of 16384 tokens exceed the L2"},
            "s_per_update": ms * 1e-3, "peak_GiB": peak_gib, "base_gemm_tflops": base_flops / (ms * 1e-3) / 1e12, "loss": final,
            "adapter_parameters": sum(p.numel() for p in lora_parameters(model)), "clocks": clk.summary()}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    cfg = dict(C3)
    res = cpu_train_baseline(cfg)
    tokens = cfg["micro_batch"] * cfg["seq"]
    return {"impl": "reference", "metric": "nvfp4_train_tokens_per_s", "value": res["value"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": tokens / res["value"] * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 arithmetic restated in FP32 on the CPU", "data": "synthetic",
            "config": {"workload": "C3 on the host cores: CPU restatement of the reference kernels (the reference itself needs an SM120 GPU "
                                   "and has no CPU path); extrapolated from one layer", "global_batch": cfg["micro_batch"], "seq_len": cfg["seq"]},
            "cpu_baseline": res, "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="train", choices=("train", "quant", "gemm", "adamw", "lora_nvfp4", "lora_packed"))
    ap.add_argument("--profiler-range", action="store_true", help="bracket the timed region with cudaProfilerStart/Stop")
    ap.add_argument("--backward-mode", default="recompute", choices=("recompute", "cache"), help="lora_packed only")
    ap.add_argument("--blocks", type=int, default=0, help="override the block count of the LoRA workloads (smoke runs only)")
    ap.add_argument("--layers", type=int, default=0, help="override the decoder depth (smoke runs only; the metric needs the default)")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    ap.add_argument("--no-variants", action="store_true", help="train workload: skip the second run with the other SR generator")
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
    runners = {"quant": run_quant, "train": run_train, "gemm": run_gemm, "adamw": run_adamw, "lora_nvfp4": run_lora, "lora_packed": run_lora}
    line = runners[args.workload](args, rank, world, device)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
