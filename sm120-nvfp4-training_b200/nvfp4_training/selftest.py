"""GPU integration check of the public training interface, after the reference's src/nvfp4_training/selftest.py: for
every requested profile, an aligned and a ragged tied-embedding model, with and without remat, run eager steps with
changing batch shapes and a captured step, and require a byte-exact continuation after save_checkpoint /
load_checkpoint into a fresh model."""
import json
import tempfile
from pathlib import Path

import torch
from torch import nn
from torch.nn import functional as F

from . import capture_step, check_finite, enable_nvfp4, list_profiles, load_checkpoint, save_checkpoint, train_step
from ._runtime import load_runtime


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


def _bytes(model):
    opt = model.nvfp4_optimizer
    out = []
    for p in model.parameters():
        out.append(p.detach().reshape(-1).view(torch.uint8).clone())
        out.extend(v.detach().reshape(-1).view(torch.uint8).clone() for _, v in sorted(opt.state.get(p, {}).items())
                   if torch.is_tensor(v))
    return out


def run_one(profile, shape, remat, folder):
    width, hidden, vocab, tokens = (512, 512, 512, 128) if shape == "aligned" else (131, 197, 257, 19)

    def build():
        torch.manual_seed(314)
        return enable_nvfp4(TinyLM(width, hidden, vocab).cuda(), profile=profile, remat=remat, lr=2e-4, betas=(.89, .995),
                            weight_decay=.02)
    rng = load_runtime()[2]
    rng.reset_stats(71)
    model = build()
    gen = torch.Generator(device="cuda").manual_seed(5)
    data = [torch.randint(0, vocab, (2, 3, tokens + i), device="cuda", generator=gen) for i in range(3)]
    losses = [train_step(model, objective, d[0], d[1]).item() for d in data]          # shapes change between eager steps
    with capture_step(model, objective, data[0][0], data[0][1], steps=2) as graph:
        losses += [graph.step(data[0][0], data[0][1]).item() for _ in range(2)]
    path = Path(folder) / f"{profile}-{shape}-{int(remat)}.pt"
    save_checkpoint(path, model)
    expected = train_step(model, objective, data[1][0], data[1][1]).item()
    other = build()
    step = load_checkpoint(path, other)
    actual = train_step(other, objective, data[1][0], data[1][1]).item()
    exact = expected == actual and all(torch.equal(a, b) for a, b in zip(_bytes(model), _bytes(other)))
    check_finite(model)
    if not exact or step != 5:
        raise RuntimeError(f"{profile}/{shape}/remat={remat}: continuation after a checkpoint is not exact")
    return dict(profile=profile, shape=shape, remat=remat, losses=losses, resumed_at=step, exact_resume=True, stats=rng.stats())


def run(profiles=None, output=None):
    profiles = tuple(profiles) if profiles else tuple(list_profiles())
    rows = []
    with tempfile.TemporaryDirectory() as folder:
        for profile in profiles:
            for shape in ("aligned", "ragged"):
                for remat in (False, True):
                    rows.append(run_one(profile, shape, remat, folder))
                    print("passed", profile, shape, "remat" if remat else "paired", flush=True)
    report = dict(status="passed", torch=torch.__version__, gpu=torch.cuda.get_device_name(), cases=rows)
    if output:
        Path(output).write_text(json.dumps(report, indent=2))
    return report
