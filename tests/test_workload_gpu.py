"""Fused element-wise workload kernels (rotary embedding, SwiGLU) against plain PyTorch FP32 references."""
import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu


def test_rope_forward_and_backward():
    from nvfp4_training._workloads.fused import rope
    from nvfp4_training._workloads.llama import apply_rotary, rotary_tables
    b, s, h, d = 2, 96, 3, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    proj = torch.randn(b, s, h * d, device="cuda", dtype=torch.bfloat16, generator=g)
    cos, sin = rotary_tables(s, d, "cuda")
    x = proj.view(b, s, h, d).clone().requires_grad_(True)
    y = rope(x, cos.contiguous(), sin.contiguous())
    xf = x.detach().float().transpose(1, 2).requires_grad_(True)
    yf = apply_rotary(xf, cos.float(), sin.float()).transpose(1, 2)
    assert torch.allclose(y.float(), yf, atol=2e-2, rtol=2e-2)
    gy = torch.randn_like(y)
    y.backward(gy)
    yf.backward(gy.float())
    assert torch.allclose(x.grad.float(), xf.grad.transpose(1, 2), atol=2e-2, rtol=2e-2)
    # rotation preserves the norm of each (a, b) pair
    assert torch.allclose(y.float().pow(2).sum(-1), x.detach().float().pow(2).sum(-1), rtol=2e-2)


def test_swiglu_forward_and_backward():
    from nvfp4_training._workloads.fused import swiglu
    g = torch.Generator(device="cuda").manual_seed(1)
    gate = (torch.randn(300, 512, device="cuda", generator=g) * 3).bfloat16().requires_grad_(True)
    up = torch.randn(300, 512, device="cuda", generator=g).bfloat16().requires_grad_(True)
    out = swiglu(gate, up)
    gf, uf = gate.detach().float().requires_grad_(True), up.detach().float().requires_grad_(True)
    ref = F.silu(gf) * uf
    assert torch.allclose(out.float(), ref, atol=1e-2, rtol=1e-2)
    d = torch.randn_like(out)
    out.backward(d)
    ref.backward(d.float())
    assert torch.allclose(gate.grad.float(), gf.grad, atol=2e-2, rtol=2e-2)
    assert torch.allclose(up.grad.float(), uf.grad, atol=2e-2, rtol=2e-2)
