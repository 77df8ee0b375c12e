"""LoRA over NVFP4 re-packed bases on the GPU (mode 'nvfp4'): training, exact resume, checkpoint recomputation, the
paired-seed input gradient, graph replay equal to eager.  Cases follow the reference's tests/test_lora.py:67-141,155-175
and tests/test_lora_graph.py:9-39."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def relative(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("mode", ["preserve", "nvfp4"])
def test_updates_resume_checkpoint_accumulation(mode, tmp_path):
    from precision_lora import prepare_lora, lora_parameters, save_lora, load_lora

    def make(checkpoint=False):
        torch.manual_seed(52)
        net = nn.Sequential(nn.Sequential(nn.Linear(129, 193), nn.GELU()), nn.Linear(193, 65)).cuda().bfloat16()
        return prepare_lora(net, mode=mode, rank=8, alpha=8, checkpoint_modules=["0"] if checkpoint else [], lr=.002)
    m, opt = make()
    frozen = {n: p.clone() for n, p in m.named_parameters() if not p.requires_grad}
    x = torch.randn(3, 17, 129, device="cuda", dtype=torch.bfloat16)
    target = torch.randn(3, 17, 65, device="cuda")

    def step(m, opt):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = (m(x).float() - target).square().mean()
        loss.backward()
        torch.nn.utils.clip_grad_norm_(lora_parameters(m), 1., error_if_nonfinite=True)
        opt.step()
        return loss.item()
    losses = [step(m, opt) for _ in range(64)]
    assert losses[-1] < losses[0] * .85, (mode, losses[0], losses[-1])
    assert all(p.grad is None and torch.equal(p, frozen[n]) for n, p in m.named_parameters() if not p.requires_grad)
    path = tmp_path / "adapter.pt"
    save_lora(path, m, optimizer=opt, base_id="test-base")
    expected_loss = step(m, opt)
    expected = [p.clone() for p in lora_parameters(m)]
    other, oo = make()
    load_lora(path, other, optimizer=oo, base_id="test-base")
    assert step(other, oo) == expected_loss
    assert all(torch.equal(a, b) for a, b in zip(expected, lora_parameters(other)))
    # recomputation inside a checkpointed block must not consume stochastic-rounding samples of the backward
    plain, po = make()
    ck, co = make(True)
    assert step(plain, po) == step(ck, co)
    assert all(torch.equal(a, b) for a, b in zip(lora_parameters(plain), lora_parameters(ck)))
    opt.zero_grad(set_to_none=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        (m(x).float().square().mean() / 2).backward()
        (m(x).float().square().mean() / 2).backward()
    assert all(torch.isfinite(p.grad).all() for p in lora_parameters(m))


def test_nvfp4_base_has_no_master_and_tracks_the_dense_layer():
    from precision_lora import enable_lora
    from precision_lora.core import _FrozenFP4
    torch.manual_seed(3)
    dense = nn.Linear(512, 384, device="cuda").bfloat16()
    x = torch.randn(64, 512, device="cuda", dtype=torch.bfloat16)
    want = dense(x)
    m = enable_lora(dense, mode="nvfp4", rank=8)
    assert isinstance(m.base, _FrozenFP4) and not list(m.base.parameters())
    assert {n for n, _ in m.base.named_buffers()} >= {"forward_data", "forward_scale", "forward_pts", "backward_data",
                                                       "backward_scale", "backward_pts", "signs", "sr_seed", "bias"}
    assert relative(m(x), want) < 0.15
    with pytest.raises(TypeError):
        with torch.autocast("cuda", dtype=torch.float16):
            m(x)


@pytest.mark.parametrize("k,n,t", [(128, 256, 64), (257, 193, 17)])
def test_paired_seed_input_gradient_equals_separate_pipeline(k, n, t):
    """dX of the LoRA layer (B = 0) is bit-equal to quantise(G, RHT, SR, seed) @ packed W for 16 seeds."""
    from precision_lora import enable_lora
    from nvfp4_training._backend import quant as backend
    torch.manual_seed(9)
    m = enable_lora(nn.Linear(k, n, device="cuda").bfloat16(), mode="nvfp4", rank=8)
    x = torch.randn(2, t, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(2, t, n, device="cuda", dtype=torch.bfloat16)
    samples = []
    before = backend.stats()
    for seed in range(16):
        m.base.sr_seed.fill_(seed)
        dx = torch.autograd.grad(m(x), x, g)[0]
        aq = backend.quantize(g.reshape(-1, n), rht=True, sr=True, signs=m.base.signs, seed=seed)
        wq = backend.Packed(m.base.backward_data, m.base.backward_scale, m.base.backward_pts, g.dtype)
        expected = backend.matmul(aq, wq, rows=2 * t, cols=k, output_dtype=g.dtype).reshape_as(x)
        assert torch.equal(dx, expected), relative(dx, expected)
        assert int(m.base.sr_seed.item()) == seed + 1
        samples.append(dx.float())
    assert not torch.equal(samples[0], samples[1]), "the SR seed must change the samples"
    after = backend.stats()
    assert after["fp4_gemm"] > before["fp4_gemm"] and after["rht_quant"] > before["rht_quant"]
    assert after["sr_quant"] > before["sr_quant"]


@pytest.mark.parametrize("mode", ["preserve", "nvfp4"])
def test_graph_replay_equals_eager(mode):
    from precision_lora import prepare_lora, capture_lora_step, lora_parameters
    from precision_lora.core import _FrozenFP4

    def make():
        torch.manual_seed(184)
        net = nn.Sequential(nn.Linear(257, 193), nn.GELU(), nn.Linear(193, 65)).cuda().bfloat16()
        return prepare_lora(net, mode=mode, rank=8, lr=.001)

    def loss_fn(m, x, y):
        return (m(x).float() - y).square().mean()
    m, opt = make()
    ref, ro = make()
    x = torch.randn(2, 17, 257, device="cuda", dtype=torch.bfloat16)
    y = torch.randn(2, 17, 65, device="cuda")
    initial = [p.detach().clone() for p in lora_parameters(m)]
    with capture_lora_step(m, opt, loss_fn, x, y) as graph:
        assert all(torch.equal(a, b) for a, b in zip(initial, lora_parameters(m))), "capture must not train"
        assert all(s["step"].item() == 0 for s in opt.state.values())
        for step in range(8):
            ro.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                expected = loss_fn(ref, x, y)
            expected.backward()
            ro.step()
            actual = graph.step(x, y)
            assert actual.item() == expected.item(), (mode, step, actual, expected)
        assert all(torch.equal(a, b) for a, b in zip(lora_parameters(m), lora_parameters(ref)))
        assert all(s["step"].item() == 8 for s in opt.state.values())
        with pytest.raises(ValueError):
            graph.step(x[:1], y[:1])
    with pytest.raises(RuntimeError):
        graph.step(x, y)
    # re-capture of a started optimizer neither resets nor advances it
    with capture_lora_step(m, opt, loss_fn, x, y) as graph:
        assert all(s["step"].item() == 8 for s in opt.state.values())
        graph.step(x, y)
    assert all(s["step"].item() == 9 for s in opt.state.values())
    seeds = [b.sr_seed.item() for b in m.modules() if isinstance(b, _FrozenFP4)]
    if seeds:
        assert seeds[-1] == 100003 + 9


def test_capture_argument_checks():
    from precision_lora import prepare_lora, capture_lora_step
    net = nn.Sequential(nn.Linear(64, 64)).cuda().bfloat16()
    m, opt = prepare_lora(net, rank=4)
    x = torch.randn(4, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="two warmup"):
        capture_lora_step(m, opt, lambda m, x: m(x).float().mean(), x, warmup=1)
    sgd = torch.optim.SGD(opt.param_groups[0]["params"], lr=0.1)
    with pytest.raises(ValueError, match="fused"):
        capture_lora_step(m, sgd, lambda m, x: m(x).float().mean(), x)
    with pytest.raises(ValueError, match="CUDA tensor"):
        capture_lora_step(m, opt, lambda m, x: m(x).float().mean(), x.cpu())
