"""Timing of full public-API training steps, with the protocol of the reference's src/nvfp4_training/benchmark.py:38-64:
the step is captured once, warmed up, then timed over rounds of synchronised steps; the report is the median of the
round means.  Task '453m' is the synthetic 16-block transformer; 'fineweb' needs a tokenised FineWeb shard that does not
ship with this package."""
import json
import statistics
import time
from pathlib import Path

import torch
from torch.nn import functional as F

from . import capture_step, check_finite, prepare_training
from ._runtime import load_runtime


def run(a):
    if a.task != "453m":
        raise RuntimeError("task 'fineweb' needs the tokenised FineWeb shard of the reference project; use --task 453m")
    torch.cuda.reset_peak_memory_stats()
    torch.manual_seed(a.seed)
    from ._workloads.synthetic import Network
    layers = 16
    model = Network(1536, layers, 12)
    gen = torch.Generator(device="cuda").manual_seed(2026)
    x, y = (torch.randn(a.batch, a.seq, 1536, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(2))

    def compute(model, x, y):
        return F.mse_loss(model(x).float(), y.float())
    model, opt = prepare_training(model, profile=a.profile, precision=a.precision, remat=a.remat)
    rng = load_runtime()[2]
    rng.reset_stats(0)
    total = a.warmup + a.rounds * a.steps
    # the attention library allocates plans and workspaces on first use, which must not happen inside a capture
    q, k, v = (torch.randn(a.batch, 12, a.seq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    F.scaled_dot_product_attention(q, k, v).float().sum().backward()
    del q, k, v
    torch.cuda.synchronize()
    graph = capture_step(model, compute, x, y, steps=total)
    times, losses = [], []
    with graph:
        linears = 4 * layers
        gemms = rng.stats()["fp4_gemm"]
        if graph.sr_calls != 2 * linears:
            raise RuntimeError(f"Unexpected stochastic-rounding count {graph.sr_calls} (expected {2 * linears})")
        for _ in range(a.warmup):
            graph.step(x, y)
        for _ in range(a.rounds):
            torch.cuda.synchronize()
            start = time.perf_counter()
            for _ in range(a.steps):
                last = graph.step(x, y)
            torch.cuda.synchronize()
            times.append(1000 * (time.perf_counter() - start) / a.steps)
            losses.append(last.item())
            if not torch.isfinite(last).item():
                raise FloatingPointError("Nonfinite training loss")
        peak = torch.cuda.max_memory_allocated() / 2 ** 30
        reserved = torch.cuda.max_memory_reserved() / 2 ** 30
    check_finite(model)
    if any(s["step"] != total for s in opt.state.values()):
        raise RuntimeError("Optimizer step count mismatch")
    ms = statistics.median(times)
    report = dict(config=vars(a), torch=torch.__version__, gpu=torch.cuda.get_device_name(), rounds_ms=times, step_ms=ms,
                  tokens_s=1000 * a.batch * a.seq / ms, train_peak_GiB=peak, train_reserved_GiB=reserved,
                  gemm_launches_until_capture=gemms, sr_calls=graph.sr_calls, losses=losses)
    if a.output:
        Path(a.output).write_text(json.dumps(report, indent=2), encoding="utf8")
    print(json.dumps(report, indent=2), flush=True)
    return report
