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
    ok = torch.tensor([int(same and losses[-1] < 0.8 * losses[0])], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"DP_RESULT ok={int(ok.item())} same={same} first={losses[0]:.4f} last={losses[-1]:.4f}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
