"""Packed-checkpoint LoRA backend on the GPU: every kernel bit for bit against the CPU oracle, then the behaviour the
reference's tests/test_packed_lora.py checks (correctly rounded backward scale, packed -> packed transpose equal to
quantise(dequantise^T), cache == recompute, paired-seed SR input gradient, AWQ input scaling, training with resume)."""
import numpy as np
import pytest
import torch
from torch import nn
from torch.nn import functional as F

import oracle as O

pytestmark = pytest.mark.gpu

LAYOUT = "comfy-high-first-swizzle128x4"


def bits(t):
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def raw(t):
    return t.detach().contiguous().reshape(-1).view(torch.uint8).cpu().numpy()


def tensor(n, k, seed, scale=0.08, outliers=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(n, k, generator=g, device="cuda", dtype=torch.bfloat16) * scale
    if outliers:
        pos = torch.randint(0, x.numel(), (max(1, x.numel() // 500),), generator=g, device="cuda")
        x.view(-1)[pos] *= 40
    return x


@pytest.mark.parametrize("rows,cols", [(1, 128), (17, 256), (128, 384), (193, 1024), (600, 512)])
@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("sr", [False, True])
def test_quantise_matches_oracle(rows, cols, rotate, sr):
    from precision_lora import _packed_cuda as cuda
    x = tensor(rows, cols, rows + cols, outliers=True)
    if rows > 3:
        x[2] = 0
    signs = torch.from_numpy(O.comfy_signs(7)).cuda() if rotate else None
    seed = 0x9E3779B1 if sr else 0
    q, s, g = cuda.quantize(x, signs, seed=seed, sr=sr)
    wq, ws, wg = O.comfy_quantize(bits(x), None if signs is None else signs.cpu().numpy(), sr=sr, seed=seed)
    assert q.shape == wq.shape and s.numel() == ws.size
    assert np.float32(g.item()) == wg
    assert np.array_equal(raw(s), ws)
    assert np.array_equal(raw(q), wq.reshape(-1))
    if sr:   # a device counter adds to the seed inside the kernel
        counter = torch.tensor(5, dtype=torch.int32, device="cuda")
        q2, _, _ = cuda.quantize(x, signs, seed=counter, sr=True)
        assert np.array_equal(raw(q2), O.comfy_quantize(bits(x), None if signs is None else signs.cpu().numpy(), sr=True, seed=5)[0].reshape(-1))


def test_zero_input_and_floor_scale():
    from precision_lora import _packed_cuda as cuda
    x = torch.zeros(16, 128, device="cuda", dtype=torch.bfloat16)
    q, s, g = cuda.quantize(x)
    assert not q.any() and not s.view(torch.uint8).any() and g.item() == np.float32(1e-30)


@pytest.mark.parametrize("n,k", [(128, 128), (256, 384), (11, 48), (130, 80)])
def test_dequantise_matches_oracle(n, k):
    from precision_lora import _packed_cuda as cuda
    rng = np.random.default_rng(n * k)
    q = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = rng.integers(0, 127, O.round128(n) * ((k + 63) // 64) * 4, dtype=np.uint8)
    g = np.float32(0.0137)
    got = cuda.dequant(torch.from_numpy(q).cuda(), torch.from_numpy(s).cuda().view(torch.float8_e4m3fn), torch.tensor(g, device="cuda"))
    assert np.array_equal(bits(got), O.comfy_dequantize(q, s, g))


@pytest.mark.parametrize("n,k", [(128, 128), (256, 384), (384, 128)])
def test_transpose_requant_matches_oracle_and_reference_relation(n, k):
    from precision_lora import _packed_cuda as cuda
    w = tensor(n, k, 11 + n, outliers=True)
    signs_np = O.comfy_signs(91)
    signs = torch.from_numpy(signs_np).cuda()
    source = cuda.quantize(w)
    bscale = cuda.backward_scale(source, signs)
    qt, st, _ = cuda.transpose_rht_quant(source, signs, bscale)
    q_np, s_np, g_np = raw(source[0]).reshape(n, k // 2), raw(source[1]), np.float32(source[2].item())
    want_scale = O.comfy_backward_scale(q_np, s_np, g_np, signs_np)
    assert np.float32(bscale.item()) == want_scale
    wqt, wst = O.comfy_transpose_requant(q_np, s_np, g_np, signs_np, want_scale)
    assert np.array_equal(raw(qt), wqt.reshape(-1)) and np.array_equal(raw(st), wst)
    # the relation the reference tests: the fused kernel equals dequantise -> transpose -> rotate + quantise
    again = cuda.quantize(cuda.dequant(*source).T.contiguous(), signs)
    assert torch.equal(again[2], bscale)
    assert torch.equal(again[0], qt) and torch.equal(again[1].view(torch.uint8), st.view(torch.uint8))


def test_finish_scale_is_correctly_rounded():
    from precision_lora import _packed_cuda as cuda
    for value in [0., 1.0872942, 1.0872943, 1., .001, 10000.]:
        amax = torch.tensor(value, dtype=torch.float32, device="cuda")
        expected = (amax.cpu().double() / 2688.).clamp_min(1e-30).float()
        assert torch.equal(cuda.finish_scale(amax).cpu(), expected)


@pytest.mark.parametrize("m,n,k", [(16, 128, 128), (48, 256, 384), (200, 128, 1024)])
def test_matmul_matches_block_scaled_product(m, n, k):
    from precision_lora import _packed_cuda as cuda
    a = cuda.quantize(tensor(m, k, 1, scale=1.0))
    b = cuda.quantize(tensor(n, k, 2, scale=0.05))
    y = cuda.matmul(a, b)
    assert y.shape == (a[0].shape[0], n) and y.dtype == torch.bfloat16

    def host(t):
        return raw(t[0]).reshape(t[0].shape[0], -1), raw(t[1]), np.float32(t[2].item())
    want = O.comfy_matmul(host(a), host(b), m, n)
    got = y[:m].float().cpu().numpy()
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 2e-3, rel          # accumulation order only; the requirement is 1e-2
    ulp = np.abs(got - want) / np.maximum(np.abs(want), 1e-30)
    assert np.quantile(ulp, 0.999) <= 2 ** -7


def test_rope_matches_oracle():
    from precision_lora import _packed_cuda as cuda
    torch.manual_seed(5)
    x = torch.randn(1, 37, 4, 32, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    rot = torch.randn(37, 12, 2, 2, device="cuda", dtype=torch.bfloat16)
    y = cuda.rope(x, rot)
    assert np.array_equal(bits(y), O.comfy_rope(bits(x), bits(rot), 12))
    g = torch.randn_like(y)
    gx = torch.autograd.grad(y, x, g)[0]
    assert np.array_equal(bits(gx), O.comfy_rope(bits(g), bits(rot), 12, backward=True))


# ---- module behaviour ----------------------------------------------------------------------------------------------
def source(n, k, seed=91):
    """A checkpoint with only the minimum scale-block padding (multiples of 16 columns), not 128-alignment."""
    from precision_lora import _packed_cuda as cuda
    from precision_lora.packed import _scale_positions as _indices
    g = torch.Generator(device="cuda").manual_seed(seed)
    full = F.pad(torch.randn(n, k, generator=g, device="cuda", dtype=torch.bfloat16) * .08, (0, -k % 128, 0, -n % 128))
    q, s, p = cuda.quantize(full)
    width = (k + 15) // 16 * 16
    small = torch.zeros(((n + 127) // 128 * 128) * ((width + 63) // 64) * 4, device="cuda", dtype=torch.uint8)
    small[_indices(n, width // 16, width, q.device)] = s.view(torch.uint8).flatten()[_indices(n, width // 16, full.shape[1], q.device)]
    return q[:n, :width // 2].contiguous(), small.view(torch.float8_e4m3fn), p


def make_base(n, k, mode="recompute", seed=91, awq=False):
    from precision_lora import PackedNVFP4Linear
    return PackedNVFP4Linear(*source(n, k, seed), shape=(n, k), layout=LAYOUT, backward_mode=mode, seed=seed,
                             input_scale=torch.linspace(.7, 1.3, k, device="cuda") if awq else None)


@pytest.mark.parametrize("n,k", [(128, 384), (193, 257), (11, 19), (256, 512)])
@pytest.mark.parametrize("awq", [False, True])
def test_padding_cache_recompute_paired_sr_awq(n, k, awq):
    from precision_lora import _packed_cuda as cuda
    torch.manual_seed(431)
    a, b = make_base(n, k, awq=awq), make_base(n, k, "cache", awq=awq)
    reference = cuda.quantize(cuda.dequant(*a.quant).T.contiguous(), a.signs)
    rebuilt = cuda.transpose_rht_quant(a.quant, a.signs, a.backward_scale)
    for u, v in zip(reference, rebuilt):
        assert torch.equal(u.reshape(-1).view(torch.uint8), v.reshape(-1).view(torch.uint8))
    for batch, seq in [(1, 1), (2, 17), (3, 64)]:
        x = torch.randn(batch, seq, k, device="cuda", dtype=torch.bfloat16).transpose(0, 1).requires_grad_()
        grad = torch.randn(n, batch, seq, device="cuda", dtype=torch.bfloat16).permute(2, 1, 0)
        ya, yb = a(x), b(x)
        assert torch.equal(ya, yb)
        ga, gb = torch.autograd.grad(ya, x, grad)[0], torch.autograd.grad(yb, x, grad)[0]
        assert torch.equal(ga, gb)
        flat = F.pad(grad.reshape(-1, n), (0, a.packed.shape[0] - n)).contiguous()
        seed = int(a.sr_seed.item()) - 1
        ref = cuda.matmul(cuda.quantize(flat, a.signs, seed=seed, sr=True), reference)[:batch * seq, :k]
        if awq:
            ref = (ref * a.input_scale).bfloat16()
        assert torch.equal(ga, ref.reshape_as(x))
        # forward against the dense product of the decoded weight
        dense_w = cuda.dequant(*a.quant)[:n, :k].float()
        xin = x.float() * a.input_scale if awq else x.float()
        want = xin @ dense_w.t()
        assert ((ya.float() - want).norm() / want.norm().clamp_min(1e-6)).item() < 0.12
    first = a.sr_seed.clone()
    g1 = torch.autograd.grad(a(x), x, grad)[0]
    g2 = torch.autograd.grad(a(x), x, grad)[0]
    assert not torch.equal(g1, g2), "SR must change between backward calls"
    a.sr_seed.copy_(first)
    assert torch.equal(torch.autograd.grad(a(x), x, grad)[0], g1), "SR repeatability"


def test_constructor_validation():
    from precision_lora import PackedNVFP4Linear
    q, s, p = source(32, 64)
    with pytest.raises(ValueError, match="layout"):
        PackedNVFP4Linear(q, s, p, layout="other")
    with pytest.raises(ValueError, match="backward_mode"):
        PackedNVFP4Linear(q, s, p, layout=LAYOUT, backward_mode="lazy")
    with pytest.raises(TypeError):
        PackedNVFP4Linear(q.cpu(), s, p, layout=LAYOUT)
    with pytest.raises(TypeError):
        PackedNVFP4Linear(q, s.view(torch.uint8), p, layout=LAYOUT)
    with pytest.raises(ValueError, match="logical shape"):
        PackedNVFP4Linear(q, s, p, layout=LAYOUT, shape=(33, 64))
    with pytest.raises(ValueError, match="scale storage"):
        PackedNVFP4Linear(q, s[:-4], p, layout=LAYOUT)
    with pytest.raises(ValueError, match="Tensor scale"):
        PackedNVFP4Linear(q, s, -p, layout=LAYOUT)
    dirty = q.clone()
    dirty[31, 0] = 0x22
    with pytest.raises(ValueError, match="row padding"):
        PackedNVFP4Linear(dirty, s, p, layout=LAYOUT, shape=(31, 64))
    with pytest.raises(ValueError, match="column padding"):
        PackedNVFP4Linear(dirty, s, p, layout=LAYOUT, shape=(32, 1))


def test_dtype_guard_autocast_and_capture_refusal():
    invalid = make_base(11, 19).bfloat16()
    with pytest.raises(TypeError):
        invalid(torch.randn(2, 19, device="cuda", dtype=torch.bfloat16))
    base = make_base(11, 19)
    x = torch.randn(2, 19, device="cuda", dtype=torch.float32, requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = base(x)
    assert y.dtype == torch.bfloat16
    y.sum().backward()
    assert x.grad.dtype == torch.float32 and torch.isfinite(x.grad).all()
    with pytest.raises(TypeError):
        base(torch.randn(2, 19, device="cuda"))   # FP32 without autocast


def test_mlp_updates_resume_checkpoint(tmp_path):
    from precision_lora import prepare_lora, lora_parameters, save_lora, load_lora, capture_lora_step

    def make(mode="recompute", checkpoint=False):
        torch.manual_seed(157)
        net = nn.Sequential(nn.Sequential(make_base(193, 129, mode), nn.GELU()), make_base(65, 193, mode, seed=93))
        return prepare_lora(net, mode="packed_nvfp4", rank=8, alpha=8, lr=.002, checkpoint_modules=["0"] if checkpoint else [])
    net, opt = make()
    cached, co = make("cache")
    ck, cko = make(checkpoint=True)
    assert net.lora_config["packed_layouts"]["1"] == dict(shape=(193, 65), layout=LAYOUT, rht_seed=93)
    x = torch.randn(3, 17, 129, device="cuda", dtype=torch.bfloat16)
    target = torch.randn(3, 17, 65, device="cuda")
    frozen = {n: t.clone() for n, t in net.named_buffers() if not n.endswith("sr_seed")}

    def step(m, o):
        o.zero_grad(set_to_none=True)
        loss = (m(x).float() - target).square().mean()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(lora_parameters(m), 1., error_if_nonfinite=True)
        o.step()
        return loss.item()
    losses = []
    for i in range(64):
        v = step(net, opt)
        losses.append(v)
        if i < 3:
            assert v == step(cached, co) == step(ck, cko)
            for p, q, r in zip(lora_parameters(net), lora_parameters(cached), lora_parameters(ck)):
                assert torch.equal(p, q) and torch.equal(p, r)
    assert losses[-1] < losses[0] * .85, losses
    for n, t in net.named_buffers():
        if n in frozen:
            assert torch.equal(t.reshape(-1).view(torch.uint8), frozen[n].reshape(-1).view(torch.uint8)), n
    path = tmp_path / "adapter.pt"
    save_lora(path, net, optimizer=opt, base_id="synthetic@91")
    expected = step(net, opt)
    restored, ro = make("cache")
    load_lora(path, restored, optimizer=ro, base_id="synthetic@91")
    assert step(restored, ro) == expected
    assert all(torch.equal(p, q) for p, q in zip(lora_parameters(net), lora_parameters(restored)))
    with pytest.raises(ValueError, match="eager"):
        capture_lora_step(net, opt, lambda m, x, y: (m(x).float() - y).square().mean(), x, target)


def test_two_block_attention_with_checkpointing():
    from precision_lora import prepare_lora, lora_parameters

    class Attention(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = make_base(384, 128)
            self.proj = make_base(128, 128, seed=17)
            self.fc1 = make_base(193, 128, seed=18)
            self.fc2 = make_base(128, 193, seed=19)

        def forward(self, x):
            q, k, v = self.qkv(F.layer_norm(x, (128,))).chunk(3, dim=-1)

            def heads(t):
                return t.reshape(*t.shape[:-1], 4, 32).transpose(1, 2)
            z = F.scaled_dot_product_attention(heads(q), heads(k), heads(v)).transpose(1, 2).reshape_as(x)
            y = x + self.proj(z)
            return y + self.fc2(F.gelu(self.fc1(F.layer_norm(y, (128,)))))
    torch.manual_seed(77)
    model, opt = prepare_lora(nn.Sequential(Attention(), Attention()), mode="packed_nvfp4", rank=8, lr=.001,
                              checkpoint_modules=["0", "1"])
    x = torch.randn(2, 37, 128, device="cuda", dtype=torch.bfloat16)
    y = torch.randn_like(x).float()
    losses = []
    for _ in range(32):
        opt.zero_grad(set_to_none=True)
        loss = (model(x).float() - y).square().mean()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(lora_parameters(model), 1., error_if_nonfinite=True)
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0], losses
