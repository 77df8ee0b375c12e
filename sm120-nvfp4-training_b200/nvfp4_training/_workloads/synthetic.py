"""Bidirectional transformer trunk of the reference's 453 M synthetic benchmark (src/nvfp4_training/_workloads/synthetic.py:
16 blocks of width 1536 with 12 heads): pre-norm blocks with a fused QKV projection, unmasked attention through PyTorch's
SDPA, a GELU feed-forward of four times the width, no biases on the projections, a final LayerNorm."""
import torch
from torch import nn
from torch.nn import functional as F


class Block(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.proj = nn.Linear(dim, dim, bias=False)
        self.up = nn.Linear(dim, 4 * dim, bias=False)
        self.down = nn.Linear(4 * dim, dim, bias=False)

    def forward(self, x):
        batch, tokens, dim = x.shape
        h = self.norm1(x).to(torch.bfloat16)
        q, k, v = self.qkv(h).view(batch, tokens, 3, self.heads, dim // self.heads).permute(2, 0, 3, 1, 4).unbind(0)
        mixed = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(batch, tokens, dim)
        x = x + self.proj(mixed)
        return x + self.down(F.gelu(self.up(self.norm2(x).to(torch.bfloat16))))


class Network(nn.Module):
    def __init__(self, dim: int, layers: int, heads: int):
        super().__init__()
        self.blocks = nn.ModuleList(Block(dim, heads) for _ in range(layers))
        self.last_norm = nn.LayerNorm(dim)

    def forward(self, x):
        for block in self.blocks:
            x = block(x)
        return self.last_norm(x)
