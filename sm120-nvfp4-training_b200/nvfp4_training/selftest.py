"""GPU integration check of the public training interface (`python -m nvfp4_training check`).

Same cases and invariants as the reference's src/nvfp4_training/selftest.py: for every requested profile, an aligned and
a ragged tied-embedding model, with and without remat,
  * the converted layers store their masters in the profile's dtype and the tied head stays FP32;
  * one captured step holds 9 NVFP4 GEMMs, 6 stochastic-rounding draws and 6 Hadamard-transformed quantisations
    (three converted layers x forward, input gradient, weight gradient);
  * replays, an eager step on a shorter batch, BF16-autocast evaluation;
  * the update after save_checkpoint / load_checkpoint into a fresh model is byte-identical, as are both state dicts;
  * the restored model can be captured again; a NaN code poked into an FP8 master is reported by check_finite.
"""
import json
import tempfile
from pathlib import Path

import torch
from torch import nn
from torch.nn import functional as F

from . import capture_step, check_finite, enable_nvfp4, list_profiles, load_checkpoint, save_checkpoint, train_step
from ._runtime import load_runtime

MASTER_DTYPE = {"balanced": torch.float16, "short128": torch.float16, "conservative": torch.bfloat16, "same_as_v5": torch.float32,
                "experimental_m4v4": torch.float16, "experimental_fp8_master": torch.float8_e4m3fn}
SHAPES = {"aligned": (512, 512, 512, 128), "ragged": (131, 197, 257, 19)}     # width, hidden, vocabulary, tokens


class TinyLM(nn.Module):
    def __init__(self, width, hidden, vocab):
        super().__init__()
        self.embedding = nn.Embedding(vocab, width)
        self.norm = nn.LayerNorm(width)
        self.up, self.down = nn.Linear(width, hidden), nn.Linear(hidden, width)
        self.head = nn.Linear(width, vocab, bias=False)
        self.head.weight = self.embedding.weight

    def forward(self, tokens):
        x = self.norm(self.embedding(tokens))
        return self.head(x + self.down(F.silu(self.up(x))))


def objective(model, x, y):
    return F.cross_entropy(model(x).flatten(0, 1).float(), y.flatten())


def _identical(a, b, where="state"):
    """Byte equality of nested containers of tensors and plain values."""
    if torch.is_tensor(a):
        ok = torch.is_tensor(b) and a.dtype == b.dtype and a.shape == b.shape and torch.equal(
            a.detach().reshape(-1).view(torch.uint8), b.detach().reshape(-1).view(torch.uint8))
    elif isinstance(a, dict):
        ok = isinstance(b, dict) and a.keys() == b.keys()
        for key in a if ok else ():
            _identical(a[key], b[key], f"{where}[{key!r}]")
    elif isinstance(a, (list, tuple)):
        ok = isinstance(b, (list, tuple)) and len(a) == len(b)
        for i, (u, v) in enumerate(zip(a, b)) if ok else ():
            _identical(u, v, f"{where}[{i}]")
    else:
        ok = a == b
    if not ok:
        raise RuntimeError(f"{where} differs after a checkpoint round trip")


def _require(cond, message):
    if not cond:
        raise RuntimeError(message)


def run_one(profile, shape, remat, folder):
    width, hidden, vocab, tokens = SHAPES[shape]
    tag = f"{profile}/{shape}/remat={remat}"

    def build():
        torch.manual_seed(314)
        net = TinyLM(width, hidden, vocab)
        if remat:
            net.cuda()          # without remat the conversion itself moves a CPU model (direct conversion)
        return enable_nvfp4(net, profile=profile, remat=remat, lr=2e-4, betas=(.89, .995), weight_decay=.02)

    counters = load_runtime()[2]
    model = build()
    opt = model.nvfp4_optimizer
    group = opt.param_groups[0]
    _require(model.head.weight is model.embedding.weight and model.head.weight.dtype == torch.float32, f"{tag}: tied head must stay FP32")
    _require(model.up.weight.dtype == MASTER_DTYPE[profile], f"{tag}: master dtype {model.up.weight.dtype}")
    _require(group["betas"] == (.89, .995) and group["weight_decay"] == .02, f"{tag}: optimizer settings were not passed on")
    gen = torch.Generator(device="cuda").manual_seed(5)
    x, y = (torch.randint(vocab, (1, tokens), device="cuda", generator=gen) for _ in range(2))
    counters.reset_stats(71)
    graph = capture_step(model, objective, x, y, steps=3)
    seen = counters.stats()
    _require((seen["fp4_gemm"], graph.sr_calls, seen["rht_quant"]) == (9, 6, 6),
             f"{tag}: a captured step holds {seen['fp4_gemm']} GEMMs / {graph.sr_calls} SR draws / {seen['rht_quant']} RHT quantisations, not 9 / 6 / 6")
    with graph:
        losses = [graph.step(x, y).item() for _ in range(3)]
    short = slice(0, tokens - 3)
    losses.append(train_step(model, objective, x[:, short].contiguous(), y[:, short].contiguous()).item())
    check_finite(model)
    _require(len(opt.state) == len(list(model.parameters())) and all(s["step"] == 4 for s in opt.state.values()), f"{tag}: step counters")
    model.eval()
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        logits = model(x)
    _require(logits.shape == (1, tokens, vocab) and bool(torch.isfinite(logits).all()), f"{tag}: evaluation under autocast")
    model.train()
    path = Path(folder) / f"{profile}-{shape}-{int(remat)}.pt"
    save_checkpoint(path, model)
    expected = train_step(model, objective, x, y)
    other = build()
    _require(load_checkpoint(path, other) == 4, f"{tag}: restored step number")
    actual = train_step(other, objective, x, y)
    _identical(actual, expected, "loss of the first update after the checkpoint")
    _identical(model.state_dict(), other.state_dict(), "model.state_dict()")
    _identical(opt.state_dict(), other.nvfp4_optimizer.state_dict(), "optimizer.state_dict()")
    with capture_step(other, objective, x, y, steps=2) as again:
        losses.extend(again.step(x, y).item() for _ in range(2))
    _require(all(s["step"] == 7 for s in other.nvfp4_optimizer.state.values()), f"{tag}: step counters after the second capture")
    check_finite(other)
    _require(all(map(lambda v: v == v and abs(v) != float("inf"), losses)), f"{tag}: non-finite loss")
    if profile == "experimental_fp8_master" and shape == "ragged" and not remat:
        with torch.no_grad():
            other.up.weight.view(torch.uint8).flatten()[0] = 127
        try:
            check_finite(other)
        except FloatingPointError as error:
            _require("up.weight" in str(error), f"{tag}: the report does not name the poisoned tensor")
        else:
            raise RuntimeError(f"{tag}: a NaN code in an FP8 master was not reported")
    return dict(profile=profile, shape=shape, remat=remat, gemms=seen["fp4_gemm"], sr=graph.sr_calls, rht=seen["rht_quant"],
                losses=losses, exact_resume=True, final_step=7)


def run(profiles=None, output=None):
    profiles = tuple(profiles) if profiles else tuple(list_profiles())
    rows = []
    with tempfile.TemporaryDirectory() as folder:
        for profile in profiles:
            for shape in SHAPES:
                for remat in (False, True):
                    rows.append(run_one(profile, shape, remat, folder))
                    print("passed", profile, shape, "remat" if remat else "paired", "GEMM/SR/RHT 9/6/6, exact resume", flush=True)
    report = dict(status="passed", torch=torch.__version__, gpu=torch.cuda.get_device_name(), cases=rows)
    if output:
        Path(output).write_text(json.dumps(report, indent=2))
    return report
