"""Llama-style decoder used as the synthetic full-parameter training workload: RMSNorm, rotary positions, SwiGLU feed
forward, causal attention through PyTorch's fused SDPA (attention stays BF16, as in the reference's workloads,
src/nvfp4_training/_workloads/lm.py:20), untied embedding and head.  Every nn.Linear is converted by enable_nvfp4.

The q / k / v projections are one Linear of 3 * dim outputs and gate / up one Linear of 2 * ffn outputs (same parameters
and arithmetic as separate layers, one tensor scale per fused weight), and the residual stream is carried as a pair
(x, delta) whose sum is formed inside the next normalisation kernel.  On CUDA with BF16 activations the element-wise work
runs on this library's fused kernels (_workloads/fused.py); `reference=True`, CPU tensors and other dtypes take plain
PyTorch operations with the same mathematics (the check of the fused path in the tests)."""
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


def _fused_ok(x, reference):
    return not reference and x.is_cuda and x.dtype == torch.bfloat16


class Block(nn.Module):
    def __init__(self, dim, heads, ffn, reference=False):
        super().__init__()
        self.heads, self.reference = heads, reference
        self.norm1, self.norm2 = RMSNorm(dim), RMSNorm(dim)
        self.qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.o = nn.Linear(dim, dim, bias=False)
        self.gate_up = nn.Linear(dim, 2 * ffn, bias=False)
        self.down = nn.Linear(ffn, dim, bias=False)

    def forward(self, x, delta, cos, sin):
        """The residual stream enters as x + delta (delta None for the first block) and leaves the same way."""
        b, s, d = x.shape
        if _fused_ok(x, self.reference):
            from .fused import add_rmsnorm, rope_attention, swiglu
            x, h = add_rmsnorm(x, delta, self.norm1.weight, self.norm1.eps)
            attn = self.o(rope_attention(self.qkv(h), cos, sin, self.heads))
            x, h = add_rmsnorm(x, attn, self.norm2.weight, self.norm2.eps)
            return x, self.down(swiglu(self.gate_up(h)))
        if delta is not None:
            x = x + delta
        q, k, v = (t.view(b, s, self.heads, d // self.heads).transpose(1, 2) for t in self.qkv(self.norm1(x)).split(d, dim=-1))
        q, k = apply_rotary(q, cos, sin), apply_rotary(k, cos, sin)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.o(a.transpose(1, 2).reshape(b, s, d))
        gate, up = self.gate_up(self.norm2(x)).chunk(2, dim=-1)
        return x, self.down(F.silu(gate) * up)


class Decoder(nn.Module):
    def __init__(self, *, layers=32, dim=3072, heads=24, ffn=8192, vocab=32000, seq=2048, std=0.02, reference=False):
        super().__init__()
        self.embed = nn.Embedding(vocab, dim)
        self.blocks = nn.ModuleList(Block(dim, heads, ffn, reference) for _ in range(layers))
        self.norm = RMSNorm(dim)
        self.head = nn.Linear(dim, vocab, bias=False)
        self.seq, self.head_dim, self.reference = seq, dim // heads, reference
        for p in self.parameters():
            if p.ndim == 2:
                nn.init.normal_(p, 0.0, std)
        self._tables = None

    def forward(self, ids):
        s = ids.shape[1]
        if self._tables is None or self._tables[0].shape[0] < s or self._tables[0].device != ids.device:
            self._tables = rotary_tables(max(s, self.seq), self.head_dim, ids.device)
        cos, sin = (t[:s].contiguous() for t in self._tables)
        x, delta = self.embed(ids).to(torch.bfloat16), None
        for block in self.blocks:
            x, delta = block(x, delta, cos, sin)
        if _fused_ok(x, self.reference):
            from .fused import add_rmsnorm
            return self.head(add_rmsnorm(x, delta, self.norm.weight, self.norm.eps)[1])
        return self.head(self.norm(x if delta is None else x + delta))


def warm_attention(model, batch, seq, device):
    """Run the attention operator once, forward and backward, with the training shapes.  Library back ends (cuDNN,
    cuBLAS) create handles, plans and workspaces on first use, in the calling thread and in autograd's worker thread;
    that must happen before a CUDA-graph capture."""
    heads = model.blocks[0].heads
    qkv = torch.randn(batch, seq, 3, heads, model.head_dim, device=device, dtype=torch.bfloat16)
    q, k, v = (qkv[:, :, i].detach().requires_grad_(True) for i in range(3))
    F.scaled_dot_product_attention(*(t.transpose(1, 2) for t in (q, k, v)), is_causal=True).float().sum().backward()
    h = torch.randn(batch * seq, 64, device=device, dtype=torch.bfloat16, requires_grad=True)
    F.cross_entropy((h @ h.t()[:, :128]).float(), torch.zeros(batch * seq, dtype=torch.long, device=device)).backward()
    torch.cuda.synchronize(device)


def token_loss(model, ids, targets):
    """Mean next-token cross-entropy.  BF16 logits on the GPU take this library's two loss kernels (no FP32 copy of the
    logits; the gradient arrives at the output projection with its amax); `reference=True` models and other inputs take
    torch's cross_entropy on an FP32 copy, as the reference's workload does."""
    logits = model(ids)
    flat = logits.reshape(-1, logits.shape[-1])
    if _fused_ok(flat, getattr(model, "reference", True)):
        from .fused import cross_entropy
        return cross_entropy(flat, targets.reshape(-1))
    return F.cross_entropy(flat.float(), targets.reshape(-1))


def linear_parameters(model) -> int:
    return sum(m.weight.numel() for m in model.modules() if isinstance(m, nn.Linear))
