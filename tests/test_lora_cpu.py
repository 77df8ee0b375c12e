"""LoRA host logic that needs no GPU: mode 'preserve' numerics, targeting rules, merge, checkpoint round trip.
Cases follow the reference's tests/test_lora.py:24-141 (preserve-only part)."""
import pytest
import torch
from torch import nn
from torch.nn import functional as F

from precision_lora.core import (enable_lora, prepare_lora, lora_parameters, LoRALinear, save_lora, load_lora, merge_lora,
                                 _LoRAFunction)


def relative(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def dense(m, x):
    return F.linear(x, m.base.weight, m.base.bias) + F.linear(F.linear(x, m.lora_A), m.lora_B) * (m.alpha / m.rank)


@pytest.mark.parametrize("shape", [(2, 64, 128, 256), (3, 17, 257, 193), (1, 7, 19, 11)])
def test_preserve_forward_and_gradients(shape):
    torch.manual_seed(431)
    b, t, k, n = shape
    original = nn.Linear(k, n)
    w = original.weight.detach().clone()
    p = original.weight
    m = enable_lora(original, rank=7, alpha=13)
    assert m.base.weight is p and torch.equal(p, w) and not p.requires_grad
    with torch.no_grad():
        m.lora_B.normal_(0, .03)
    x = torch.randn(b, t, k, requires_grad=True).transpose(0, 1)     # non-contiguous input and gradient
    g = torch.randn(n, b, t).permute(2, 1, 0)
    y, expected = m(x), dense(m, x)
    got = torch.autograd.grad(y, (x, m.lora_A, m.lora_B), g)
    ref = torch.autograd.grad(expected, (x, m.lora_A, m.lora_B), g)
    assert max([relative(y, expected)] + [relative(a, b) for a, b in zip(got, ref)]) < 2e-5
    assert p.grad is None and torch.equal(p, w)


def test_finite_difference_gradients():
    torch.manual_seed(0)
    base = nn.Linear(5, 7, dtype=torch.float64).requires_grad_(False)
    x = torch.randn(3, 5, dtype=torch.float64, requires_grad=True)
    a = torch.randn(2, 5, dtype=torch.float64, requires_grad=True)
    b = torch.randn(7, 2, dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda x, a, b: _LoRAFunction.apply(x, a, b, base, .7), (x, a, b))


def test_merge_keeps_dtype_and_values():
    torch.manual_seed(1)
    m = enable_lora(nn.Linear(33, 27), rank=4, alpha=9)
    with torch.no_grad():
        m.lora_B.normal_()
    x = torch.randn(8, 33)
    y = m(x).detach()
    merged = merge_lora(m)
    assert type(merged) is nn.Linear and relative(merged(x), y) < 2e-6


def test_default_targets_protect_tied_head_and_typos_change_nothing():
    shell = nn.Module()
    shell.embed = nn.Embedding(32, 16)
    shell.head = nn.Linear(16, 32, bias=False)
    shell.head.weight = shell.embed.weight
    shell.proj = nn.Linear(16, 16)
    enable_lora(shell)
    assert type(shell.head) is nn.Linear and isinstance(shell.proj, LoRALinear) and shell.head.weight is shell.embed.weight
    m = nn.Sequential(nn.Linear(4, 4))
    with pytest.raises(ValueError):
        enable_lora(m, target_modules=["typo"])
    assert all(p.requires_grad for p in m.parameters())


def test_argument_validation():
    with pytest.raises(ValueError):
        enable_lora(nn.Linear(4, 4), mode="int4")
    with pytest.raises(ValueError):
        enable_lora(nn.Linear(4, 4), rank=0)
    with pytest.raises(ValueError):
        enable_lora(nn.Linear(4, 4), alpha=float("inf"))
    with pytest.raises(TypeError):
        enable_lora(nn.Linear(4, 4), target_modules="0")
    with pytest.raises(TypeError):
        enable_lora(nn.Sequential(nn.Linear(4, 4)), mode="packed_nvfp4", target_modules=["0"])
    with pytest.raises(ValueError):   # NVFP4 bases need CUDA weights
        enable_lora(nn.Sequential(nn.Linear(4, 4)), mode="nvfp4")
    net = nn.Sequential(nn.Sequential(nn.Linear(4, 4)), nn.Linear(4, 4))
    with pytest.raises(ValueError):
        enable_lora(net, checkpoint_modules=["0", "0.0"])
    with pytest.raises(ValueError):
        prepare_lora(nn.Linear(4, 4), lr=-1)
    with pytest.raises(ValueError):
        prepare_lora(nn.Linear(4, 4), betas=(0.9, 1.0))


def test_training_checkpoint_and_resume(tmp_path):
    def make(checkpoint=False):
        torch.manual_seed(52)
        net = nn.Sequential(nn.Sequential(nn.Linear(29, 33), nn.GELU()), nn.Linear(33, 9))
        return prepare_lora(net, rank=4, alpha=4, lr=.01, checkpoint_modules=["0"] if checkpoint else [])
    m, opt = make()
    assert m.lora_config["targets"] == ["0.0", "1"]
    x, target = torch.randn(6, 29), torch.randn(6, 9)

    def step(m, opt):
        opt.zero_grad(set_to_none=True)
        loss = (m(x) - target).square().mean()
        loss.backward()
        opt.step()
        return loss.item()
    losses = [step(m, opt) for _ in range(40)]
    assert losses[-1] < losses[0]
    path = tmp_path / "adapter.pt"
    save_lora(path, m, optimizer=opt, base_id="base-1")
    expected = step(m, opt)
    other, oo = make()
    with pytest.raises(ValueError):
        load_lora(path, other, optimizer=oo, base_id="another-base")
    assert load_lora(path, other, optimizer=oo, base_id="base-1") == "base-1"
    assert step(other, oo) == expected
    assert all(torch.equal(a, b) for a, b in zip(lora_parameters(m), lora_parameters(other)))
    plain, po = make()
    ck, co = make(True)
    assert step(plain, po) == step(ck, co)
