"""Fused element-wise workload kernels (residual add + RMSNorm, rotary attention over a fused projection, SwiGLU) against
plain PyTorch FP32 references, and the amax hand-off to the quantiser against the separate amax pass."""
import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu


def _close(got, want, tol=2e-2):
    got, want = got.float(), want.float()
    assert torch.allclose(got, want, atol=tol * max(1.0, want.abs().max().item()) * 0.5, rtol=tol), (got - want).abs().max().item()


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


def test_swiglu_forward_backward_and_amax():
    from nvfp4_training._backend.quant import known_amax
    from nvfp4_training._workloads.fused import swiglu
    g = torch.Generator(device="cuda").manual_seed(1)
    gu = (torch.randn(300, 1024, device="cuda", generator=g) * 2).bfloat16().requires_grad_(True)
    out = swiglu(gu)
    ref_in = gu.detach().float().requires_grad_(True)
    gate, up = ref_in.chunk(2, dim=-1)
    ref = F.silu(gate) * up
    assert torch.allclose(out.float(), ref, atol=1e-2, rtol=1e-2)
    assert known_amax(out)[0].item() == out.detach().abs().max().item()
    d = torch.randn_like(out)
    seen = {}
    gu.register_hook(lambda grad: seen.update(amax=known_amax(grad)))
    out.backward(d)
    ref.backward(d.float())
    assert torch.allclose(gu.grad.float(), ref_in.grad, atol=2e-2, rtol=2e-2)
    assert seen["amax"] is not None and seen["amax"][0].item() == gu.grad.abs().max().item()


@pytest.mark.parametrize("rows,cols", [(64, 256), (300, 3072), (17, 8192)])
@pytest.mark.parametrize("with_delta", [True, False])
def test_add_rmsnorm_forward_backward_and_amax(rows, cols, with_delta):
    from nvfp4_training._backend.quant import known_amax
    from nvfp4_training._workloads.fused import add_rmsnorm
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16().requires_grad_(True)
    delta = (torch.randn(rows, cols, device="cuda", generator=g) * 0.5).bfloat16().requires_grad_(True) if with_delta else None
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).requires_grad_(True)
    total, h = add_rmsnorm(x, delta, gamma, 1e-5)
    xf = x.detach().float().requires_grad_(True)
    df = delta.detach().float().requires_grad_(True) if with_delta else None
    gf = gamma.detach().clone().requires_grad_(True)
    tf = xf + df if with_delta else xf   # the kernel's one extra rounding of the sum is inside the tolerance
    hf = F.rms_norm(tf, (cols,), gf.detach().bfloat16().float() + (gf - gf.detach()), 1e-5)   # value bf16(gamma), gradient to gamma
    _close(total, tf)
    _close(h, hf)
    assert known_amax(h)[0].item() == h.detach().abs().max().item()
    # gradient through both outputs: h feeds a layer, the sum continues on the residual path
    dh = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
    dt = (torch.randn(rows, cols, device="cuda", generator=g) * 0.3).bfloat16()
    seen = {}
    x.register_hook(lambda grad: seen.update(amax=known_amax(grad)))
    torch.autograd.backward([h, total], [dh, dt])
    torch.autograd.backward([hf, tf], [dh.float(), dt.float()])
    _close(x.grad, xf.grad)
    if with_delta:
        _close(delta.grad, df.grad)
        assert torch.equal(delta.grad, x.grad)
    assert torch.allclose(gamma.grad, gf.grad, rtol=2e-2, atol=2e-2 * gf.grad.abs().max().item())
    assert seen["amax"] is not None and seen["amax"][0].item() == x.grad.abs().max().item()


def test_quantiser_with_a_produced_amax_equals_the_two_pass_form(native):
    """quantize_tile_amax: scales computed inside the quantiser from a device amax == amax kernel + quantiser."""
    from _util import alloc_packing, signs_dev
    x = (torch.randn(256, 384, device="cuda") * 3).bfloat16()
    signs = signs_dev()
    want = native.amax(x)
    outs = []
    for produced in (False, True):
        slot = torch.zeros(4, device="cuda")
        slot[0] = x.abs().max().float()
        scales = slot if produced else want
        rp, rs = alloc_packing(256, 384)
        cp, cs = alloc_packing(384, 256)
        native.quantize_tile(x, signs, row=dict(packed=rp, scales=rs, pts=scales[1:2], flags=4, seed=11),
                             col=dict(packed=cp, scales=cs, pts=scales[2:3], flags=4 | 1, seed=12),
                             amax=scales[0:1] if produced else None)
        outs.append((rp, rs, cp, cs, scales[:3].clone()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_fused_decoder_matches_the_plain_pytorch_decoder():
    """Same weights, same tokens: the decoder on the fused kernels against its plain PyTorch form (both BF16, dense
    layers): loss and gradients agree to BF16 accuracy."""
    from nvfp4_training._workloads.llama import Decoder, token_loss
    cfg = dict(layers=2, dim=256, heads=2, ffn=512, vocab=512, seq=128)
    torch.manual_seed(0)
    fused = Decoder(**cfg).cuda().bfloat16()
    plain = Decoder(**cfg, reference=True).cuda().bfloat16()
    plain.load_state_dict(fused.state_dict())
    for m in (fused, plain):       # the gains stay FP32 in training; here only their values matter
        for p in m.parameters():
            p.data = p.data.float() if p.ndim == 1 else p.data
    ids = torch.randint(0, 512, (4, 129), device="cuda")
    losses = []
    for m in (fused, plain):
        loss = token_loss(m, ids[:, :-1], ids[:, 1:])
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 2e-2 * abs(losses[1])
    for (name, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        rel = (a.grad.float() - b.grad.float()).norm() / b.grad.float().norm().clamp_min(1e-12)
        assert rel < 0.06, (name, rel.item())


@pytest.mark.parametrize("rows,cols,pitch", [(1000, 32000, 32000), (513, 2048, 2048), (64, 4096, 4352), (7, 8, 8)])
def test_cross_entropy_matches_torch_on_the_fp32_copy(rows, cols, pitch):
    """Loss within FP32 rounding of torch's cross_entropy on logits.float(); gradient equal to torch's FP32 gradient rounded
    to BF16 up to one BF16 ulp (the two exp implementations may differ in the last FP32 bits); amax of the gradient left
    on the device; a scaled upstream gradient is applied inside the kernel."""
    from nvfp4_training._backend import quant
    from nvfp4_training._workloads import fused
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    store = (torch.randn(rows, pitch, device="cuda", generator=g) * 3).bfloat16()
    targets = torch.randint(0, cols, (rows,), device="cuda", generator=g)
    got_in = store[:, :cols].detach().requires_grad_(True)
    want_in = store[:, :cols].detach().clone().requires_grad_(True)
    hook = {}
    got_in.register_hook(lambda grad: hook.update(amax=quant.known_amax(grad)))
    loss = fused.cross_entropy(got_in, targets)
    (loss * 3).backward()
    want = F.cross_entropy(want_in.float(), targets)
    (want * 3).backward()
    assert abs(loss.item() - want.item()) <= 2e-6 * abs(want.item())
    a, b = got_in.grad.float(), want_in.grad.float()
    assert got_in.grad.dtype == torch.bfloat16
    ulp = b.abs().clamp_min(1e-30) * 2.0 ** -7
    assert bool(((a - b).abs() <= ulp).all())
    assert float((a != b).float().mean()) < 0.02
    if hook.get("amax") is not None:
        assert hook["amax"][0].item() == a.abs().max().item()
