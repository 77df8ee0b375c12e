"""Worker of the two-GPU data-parallel test (launched by torch.distributed.run from test_dp_gpu.py)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "sm120-nvfp4-training_b200"))


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import nvfp4_training as nv
    torch.manual_seed(100 + rank)    # different initial weights on purpose: enable_data_parallel must broadcast rank 0's
    model = nn.Sequential(nn.Linear(512, 1024), nn.GELU(), nn.LayerNorm(1024), nn.Linear(1024, 512, bias=False)).to(dev)
    model = nv.enable_nvfp4(model, profile="balanced", lr=2e-3, betas=(0.9, 0.95))
    nv.enable_data_parallel(model)

    def mse(m, x, y):
        return F.mse_loss(m(x).float(), y.float())

    g = torch.Generator(device=dev).manual_seed(7 + rank)        # every rank trains on its own shard
    x = torch.randn(256, 512, device=dev, dtype=torch.bfloat16, generator=g)
    y = torch.randn(256, 512, device=dev, dtype=torch.bfloat16, generator=g)
    losses = [nv.train_step(model, mse, x, y).item() for _ in range(20)]
    with nv.capture_step(model, mse, x, y, steps=10) as graph:
        losses += [graph.step(x, y).item() for _ in range(10)]
    nv.check_finite(model)
    # replicas must hold identical weights and optimizer state
    flat = torch.cat([p.detach().float().flatten() for p in model.parameters()] +
                     [v.float().flatten() for p in model.parameters() for k, v in sorted(model.nvfp4_optimizer.state[p].items()) if torch.is_tensor(v)])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    same = torch.equal(flat, ref)
    # a head tied to the embedding: the shared weight has a deferred NVFP4 gradient (the head) AND an autograd gradient
    # (the embedding); both must be reduced or the replicas drift apart
    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            self.embedding = nn.Embedding(256, 128)
            self.mid = nn.Linear(128, 128)
            self.head = nn.Linear(128, 256, bias=False)
            self.head.weight = self.embedding.weight

        def forward(self, tokens):
            return self.head(F.gelu(self.mid(self.embedding(tokens))))

    torch.manual_seed(300 + rank)
    tied = nv.enable_nvfp4(Tied().to(dev), profile="balanced", lr=2e-3)
    nv.enable_data_parallel(tied)

    def ce(m, t, y):
        return F.cross_entropy(m(t).flatten(0, 1).float(), y.flatten())

    tok = torch.randint(0, 256, (2, 4, 64), device=dev, generator=g)
    tied_losses = [nv.train_step(tied, ce, tok[0], tok[1]).item() for _ in range(6)]
    with nv.capture_step(tied, ce, tok[0], tok[1], steps=6) as graph:
        tied_losses += [graph.step(tok[0], tok[1]).item() for _ in range(6)]
    tflat = torch.cat([p.detach().float().flatten() for p in tied.parameters()])
    tref = tflat.clone()
    dist.broadcast(tref, src=0)
    same_tied = torch.equal(tflat, tref)
    ok = torch.tensor([int(same and same_tied and losses[-1] < 0.8 * losses[0])], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"DP_RESULT ok={int(ok.item())} same={same} same_tied={same_tied} first={losses[0]:.4f} last={losses[-1]:.4f} "
              f"tied_first={tied_losses[0]:.4f} tied_last={tied_losses[-1]:.4f}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
