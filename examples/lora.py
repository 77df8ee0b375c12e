"""LoRA over bases re-packed to NVFP4 (mode 'nvfp4'): a captured update, then an adapter checkpoint round trip."""
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "sm120-nvfp4-training_b200"))

import torch
from torch import nn

from nvfp4_training import capture_lora_step, load_lora, lora_parameters, prepare_lora, save_lora


def build(mode):
    torch.manual_seed(3)
    net = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 64)).cuda().bfloat16()
    return prepare_lora(net, mode=mode, rank=8, lr=1e-3)


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "nvfp4"
    model, opt = build(mode)
    x = torch.randn(4, 32, 256, device="cuda", dtype=torch.bfloat16)
    y = torch.randn(4, 32, 64, device="cuda")

    def loss_fn(m, x, y):
        return (m(x).float() - y).square().mean()
    with capture_lora_step(model, opt, loss_fn, x, y) as graph:
        losses = [graph.step(x, y).item() for _ in range(16)]
    print(mode, "adapter parameters", sum(p.numel() for p in lora_parameters(model)), "loss", losses[0], "->", losses[-1])
    with tempfile.TemporaryDirectory() as folder:
        path = Path(folder) / "adapter.pt"
        save_lora(path, model, optimizer=opt, base_id="example")
        other, other_opt = build(mode)
        load_lora(path, other, optimizer=other_opt, base_id="example")
        same = all(torch.equal(a, b) for a, b in zip(lora_parameters(model), lora_parameters(other)))
        print("restored adapters identical:", same)


if __name__ == "__main__":
    main()
