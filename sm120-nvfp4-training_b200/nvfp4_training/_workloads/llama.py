"""Llama-style decoder used as the synthetic full-parameter training workload: RMSNorm, rotary positions, SwiGLU feed
forward, causal attention through PyTorch's fused SDPA (attention stays BF16, as in the reference's workloads,
src/nvfp4_training/_workloads/lm.py:20), untied embedding and head.  Every nn.Linear is converted by enable_nvfp4."""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight.to(x.dtype), self.eps)


def rotary_tables(seq, head_dim, device, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, device=device, dtype=torch.float32), inv)
    return ang.cos().bfloat16(), ang.sin().bfloat16()


def apply_rotary(x, cos, sin):
    # x [B, H, S, D]; split-half rotation
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)


class Block(nn.Module):
    def __init__(self, dim, heads, ffn):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = RMSNorm(dim), RMSNorm(dim)
        self.q, self.k, self.v, self.o = (nn.Linear(dim, dim, bias=False) for _ in range(4))
        self.gate, self.up = nn.Linear(dim, ffn, bias=False), nn.Linear(dim, ffn, bias=False)
        self.down = nn.Linear(ffn, dim, bias=False)

    def forward(self, x, cos, sin):
        b, s, d = x.shape
        h = self.norm1(x)
        q, k, v = (f(h).view(b, s, self.heads, d // self.heads) for f in (self.q, self.k, self.v))
        if x.is_cuda and x.dtype == torch.bfloat16:
            from .fused import rope, swiglu
            q, k = rope(q, cos[:s], sin[:s]), rope(k, cos[:s], sin[:s])
        else:
            swiglu = lambda g, u: F.silu(g) * u
            q, k = (apply_rotary(t.transpose(1, 2), cos, sin).transpose(1, 2) for t in (q, k))
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(b, s, d))
        h = self.norm2(x)
        return x + self.down(swiglu(self.gate(h), self.up(h)))


class Decoder(nn.Module):
    def __init__(self, *, layers=32, dim=3072, heads=24, ffn=8192, vocab=32000, seq=2048, std=0.02):
        super().__init__()
        self.embed = nn.Embedding(vocab, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, ffn) for _ in range(layers))
        self.norm = RMSNorm(dim)
        self.head = nn.Linear(dim, vocab, bias=False)
        self.seq, self.head_dim = seq, dim // heads
        for p in self.parameters():
            if p.ndim == 2:
                nn.init.normal_(p, 0.0, std)
        self._tables = None

    def forward(self, ids):
        s = ids.shape[1]
        if self._tables is None or self._tables[0].shape[0] < s or self._tables[0].device != ids.device:
            self._tables = rotary_tables(max(s, self.seq), self.head_dim, ids.device)
        cos, sin = (t[:s].contiguous() for t in self._tables)
        x = self.embed(ids).to(torch.bfloat16)
        for block in self.blocks:
            x = block(x, cos, sin)
        return self.head(self.norm(x))


def warm_attention(model, batch, seq, device):
    """Run the attention operator once, forward and backward, with the training shapes.  Library back ends (cuDNN,
    cuBLAS) create handles, plans and workspaces on first use, in the calling thread and in autograd's worker thread;
    that must happen before a CUDA-graph capture."""
    heads = model.blocks[0].heads
    q, k, v = (torch.randn(batch, heads, seq, model.head_dim, device=device, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    F.scaled_dot_product_attention(q, k, v, is_causal=True).float().sum().backward()
    h = torch.randn(batch * seq, 64, device=device, dtype=torch.bfloat16, requires_grad=True)
    F.cross_entropy((h @ h.t()[:, :128]).float(), torch.zeros(batch * seq, dtype=torch.long, device=device)).backward()
    torch.cuda.synchronize(device)


def token_loss(model, ids, targets):
    logits = model(ids)
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.view(-1))


def linear_parameters(model) -> int:
    return sum(m.weight.numel() for m in model.modules() if isinstance(m, nn.Linear))
