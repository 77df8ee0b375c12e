"""Synthetic module trees for the two LoRA benchmark configurations.

GPT2Small  the GPT-2-small layout (12 blocks, width 768, 12 heads, feed-forward 3072, vocabulary 50257, learned
           positions, tied head) with random weights; LoRA targets are attn.qkv / attn.proj / mlp.up / mlp.down.
DiT        a joint text + image diffusion-transformer trunk (24 blocks, width 3072, 24 heads, GELU feed-forward 12288)
           whose four projections per block are PackedNVFP4Linear modules built from random weights quantised once
           into the packed checkpoint layout; norms, modulation-free residual blocks, no pretrained weights.
Both stand in for the pretrained models of the reference's examples (GPT-2 124M, FLUX.2 Klein), which need downloads.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F


class _GPTAttention(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4).unbind(0)
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        return self.proj(y.transpose(1, 2).reshape(b, s, d))


class _GPTMLP(nn.Module):
    def __init__(self, dim, hidden):
        super().__init__()
        self.up, self.down = nn.Linear(dim, hidden), nn.Linear(hidden, dim)

    def forward(self, x):
        return self.down(F.gelu(self.up(x), approximate="tanh"))


class _GPTBlock(nn.Module):
    def __init__(self, dim, heads, hidden):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.attn, self.mlp = _GPTAttention(dim, heads), _GPTMLP(dim, hidden)

    def forward(self, x):
        x = x + self.attn(self.ln1(x))
        return x + self.mlp(self.ln2(x))


class GPT2Small(nn.Module):
    def __init__(self, *, layers=12, dim=768, heads=12, hidden=3072, vocab=50257, positions=1024, std=0.02):
        super().__init__()
        self.wte, self.wpe = nn.Embedding(vocab, dim), nn.Embedding(positions, dim)
        self.blocks = nn.ModuleList(_GPTBlock(dim, heads, hidden) for _ in range(layers))
        self.ln = nn.LayerNorm(dim)
        self.lm_head = nn.Linear(dim, vocab, bias=False)
        self.lm_head.weight = self.wte.weight
        for p in self.parameters():
            if p.ndim == 2:
                nn.init.normal_(p, 0.0, std)

    def forward(self, ids):
        pos = torch.arange(ids.shape[1], device=ids.device)
        x = self.wte(ids) + self.wpe(pos)
        for block in self.blocks:
            x = block(x)
        return self.lm_head(self.ln(x))


GPT2_TARGETS = ["qkv", "proj", "up", "down"]


def lm_loss(model, ids, labels):
    logits = model(ids)
    return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1))


def packed_linear(out_features, in_features, *, seed, backward_mode, device, std=0.02):
    """Random weights quantised once into the packed checkpoint layout (the role of a downloaded NVFP4 checkpoint)."""
    from precision_lora import PackedNVFP4Linear, _packed_cuda as cuda
    g = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn(out_features, in_features, generator=g, device=device) * std).bfloat16()
    pad = F.pad(w, (0, -in_features % 128, 0, -out_features % 128))
    q, s, p = cuda.quantize(pad)
    return PackedNVFP4Linear(q.contiguous(), s, p, shape=(out_features, in_features), layout="comfy-high-first-swizzle128x4",
                             backward_mode=backward_mode, seed=seed)


class _DiTBlock(nn.Module):
    def __init__(self, dim, heads, hidden, make):
        super().__init__()
        self.heads = heads
        self.norm1, self.norm2 = nn.LayerNorm(dim, elementwise_affine=False), nn.LayerNorm(dim, elementwise_affine=False)
        self.qkv, self.out = make(3 * dim, dim), make(dim, dim)
        self.up, self.down = make(hidden, dim), make(dim, hidden)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(self.norm1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4).unbind(0)
        y = F.scaled_dot_product_attention(q, k, v)
        x = x + self.out(y.transpose(1, 2).reshape(b, s, d))
        return x + self.down(F.gelu(self.up(self.norm2(x)), approximate="tanh"))


class DiT(nn.Module):
    """Joint attention over [text tokens ; image tokens]; the loss is taken on the image tokens."""

    def __init__(self, *, blocks=24, dim=3072, heads=24, hidden=12288, backward_mode="recompute", device="cuda", seed=11):
        super().__init__()
        counter = [seed * 1000]

        def make(n, k):
            counter[0] += 1
            return packed_linear(n, k, seed=counter[0], backward_mode=backward_mode, device=device)
        self.blocks = nn.ModuleList(_DiTBlock(dim, heads, hidden, make) for _ in range(blocks))
        self.norm = nn.LayerNorm(dim, elementwise_affine=False)

    def forward(self, latents, text):
        x = torch.cat((text, latents), dim=1)
        for block in self.blocks:
            x = block(x)
        return self.norm(x)[:, text.shape[1]:]


DIT_TARGETS = ["qkv", "out", "up", "down"]


def denoise_loss(model, latents, text, target):
    return (model(latents, text).float() - target).square().mean()
