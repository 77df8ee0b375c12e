"""A frozen backbone stored only as NVFP4 between two trainable layers, replayed as a CUDA graph (no optimizer here)."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "sm120-nvfp4-training_b200"))

import torch
from torch import nn
from torch.nn import functional as F

from nvfp4_training import capture_frozen, pack_frozen_layers


class Example(nn.Module):
    def __init__(self):
        super().__init__()
        self.input = nn.Linear(256, 256)
        self.backbone = nn.Linear(256, 256).requires_grad_(False)
        self.output = nn.Linear(256, 8)

    def forward(self, x):
        return self.output(F.silu(self.backbone(self.input(x))))


def main():
    torch.manual_seed(7)
    model = pack_frozen_layers(Example().cuda(), include=("backbone",), keep=("input", "output"))
    x = torch.randn(8, 256, device="cuda")
    target = torch.randn(8, 8, device="cuda")

    def objective(model, x, target):
        return F.mse_loss(model(x).float(), target)
    with capture_frozen(model, objective, x, target) as replay:
        for _ in range(3):
            print("loss:", replay.replay(x, target).item(), "stochastic-rounding calls per replay:", replay.sr_calls)
    print("gradients of the trainable layers are in .grad; no optimizer step was taken")


if __name__ == "__main__":
    main()
