"""End-to-end checks of the nvfp4_training interface on a GPU: the six profiles, eager steps with changing shapes, graph
capture vs eager, exact checkpoint resume, op counters.  Modelled on the reference's self-test
(src/nvfp4_training/selftest.py:35-124) and public-usage gate (_verification/verify_fast_v2.py:223-274)."""
import copy
import io

import pytest
import torch
from torch import nn
from torch.nn import functional as F

pytestmark = pytest.mark.gpu


def make_model(d=512, hidden=1024, out=256, seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(d, hidden), nn.GELU(), nn.LayerNorm(hidden), nn.Linear(hidden, hidden, bias=False), nn.GELU(),
                         nn.Linear(hidden, out))


def mse(model, x, y):
    return F.mse_loss(model(x).float(), y.float())


def batch(tokens, d=512, out=256, seed=1):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(tokens, d, device="cuda", dtype=torch.bfloat16, generator=g),
            torch.randn(tokens, out, device="cuda", dtype=torch.bfloat16, generator=g))


def state_bytes(model):
    opt = model.nvfp4_optimizer
    out = []
    for name, p in model.named_parameters():
        out.append(p.detach().view(torch.uint8).flatten().clone() if p.dtype == torch.float8_e4m3fn else p.detach().clone())
        for key, v in sorted(opt.state.get(p, {}).items()):
            if torch.is_tensor(v):
                out.append(v.clone())
    return out


def same(a, b):
    return len(a) == len(b) and all(x.dtype == y.dtype and torch.equal(x.view(torch.uint8) if x.dtype != torch.uint8 else x,
                                                                       y.view(torch.uint8) if y.dtype != torch.uint8 else y)
                                    for x, y in zip(a, b))


STORAGE = {"balanced": torch.float16, "short128": torch.float16, "conservative": torch.bfloat16, "same_as_v5": torch.float32,
           "experimental_m4v4": torch.float16, "experimental_fp8_master": torch.float8_e4m3fn}


@pytest.mark.parametrize("profile", list(STORAGE))
@pytest.mark.parametrize("remat", [False, True])
def test_profiles_train_and_resume_exactly(profile, remat, tmp_path):
    import nvfp4_training as nv
    from nvfp4_training._runtime import load_runtime
    rng = load_runtime()[2]
    rng.reset_stats(11)
    model = nv.enable_nvfp4(make_model().cuda(), profile=profile, remat=remat, lr=1e-3)
    assert model[0].weight.dtype == STORAGE[profile] and model.nvfp4_profile == profile
    losses = []
    for tokens in (128, 131, 19):   # aligned and padded token counts
        x, y = batch(tokens, seed=tokens)
        losses.append(nv.train_step(model, mse, x, y).item())
    nv.check_finite(model)
    st = rng.stats()
    assert st["fp4_gemm"] == 3 * 3 * 3 - 3      # 3 steps x 3 layers x 3 GEMMs, no dX for the first layer
    assert st["sr_quant"] > 0 and st["rht_quant"] > 0
    path = tmp_path / "ckpt.pt"
    nv.save_checkpoint(path, model)
    x, y = batch(197, seed=5)
    nv.train_step(model, mse, x, y)
    after = state_bytes(model)
    fresh = nv.enable_nvfp4(make_model(seed=3).cuda(), profile=profile, remat=remat, lr=1e-3)
    assert nv.load_checkpoint(path, fresh) == 3
    nv.train_step(fresh, mse, x, y)
    assert same(after, state_bytes(fresh)), "update after resume is not bit-identical"


def test_loss_decreases_and_matches_bf16_direction():
    import nvfp4_training as nv
    model = nv.enable_nvfp4(make_model().cuda(), profile="balanced", lr=2e-3, betas=(0.9, 0.95))
    x, y = batch(512, seed=9)
    first = nv.train_step(model, mse, x, y).item()
    for _ in range(60):
        last = nv.train_step(model, mse, x, y).item()
    assert last < 0.5 * first
    nv.check_finite(model)


@pytest.mark.parametrize("overlap", [True, False])
def test_captured_steps_equal_eager_steps(overlap):
    """overlap: optimizer updates recorded on a second stream beside the main line (the default) or in line."""
    import nvfp4_training as nv
    from nvfp4_training._runtime import load_runtime
    rng = load_runtime()[2]
    x, y = batch(256, seed=2)
    rng.reset_stats(100)
    eager = nv.enable_nvfp4(make_model().cuda(), profile="balanced", lr=1e-3)
    for _ in range(3):
        nv.train_step(eager, mse, x, y)
    rng.reset_stats(100)
    graphed = nv.enable_nvfp4(make_model().cuda(), profile="balanced", lr=1e-3)
    graphed.nvfp4_optimizer.overlap_updates = overlap
    with nv.capture_step(graphed, mse, x, y, steps=3) as graph:
        assert graph.sr_calls == 2 * 3 - 1 + 0 or graph.sr_calls > 0
        for _ in range(3):
            loss = graph.step(x, y)
        with pytest.raises(RuntimeError):
            graph.step(x, y)
    assert torch.isfinite(loss).item()
    assert same(state_bytes(eager), state_bytes(graphed)), "graph replay diverged from eager updates"
    # eager training continues after the graph is closed, with another token count
    x2, y2 = batch(77, seed=4)
    nv.train_step(graphed, mse, x2, y2)
    nv.check_finite(graphed)


def test_argument_validation_matches_reference_errors():
    import nvfp4_training as nv
    with pytest.raises(ValueError):
        nv.enable_nvfp4(make_model().cuda(), profile="nope")
    with pytest.raises(ValueError):
        nv.prepare_training(make_model().cuda(), remat=True, precision="bf16")
    with pytest.raises(ValueError):
        nv.prepare_training(nn.Sequential(nn.GELU()).cuda())
    m = nv.enable_nvfp4(make_model().cuda())
    with pytest.raises(ValueError):
        nv.enable_nvfp4(m)
    with pytest.raises(TypeError):
        m(torch.randn(4, 512, device="cuda", dtype=torch.float64))
    with pytest.raises(ValueError):
        nv.capture_step(m, mse, *batch(128), steps=0)


def test_small_decoder_trains():
    import nvfp4_training as nv
    from nvfp4_training._workloads.llama import Decoder, token_loss
    torch.manual_seed(0)
    model = Decoder(layers=2, dim=256, heads=2, ffn=512, vocab=512, seq=128).cuda()
    model = nv.enable_nvfp4(model, profile="balanced", lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.randint(0, 512, (4, 129), device="cuda", generator=g)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    first = nv.train_step(model, token_loss, x, y).item()
    for _ in range(40):
        last = nv.train_step(model, token_loss, x, y).item()
    assert last < 0.7 * first
    nv.check_finite(model)


def test_layers_sharing_an_input_reuse_its_packing_and_edits_invalidate_it():
    """Round-to-nearest activation pairs are deterministic, so consecutive layers reading one tensor share them; the
    entry must die with an in-place edit of the source, and stochastic pairs are never shared."""
    from nvfp4_training._backend import quant
    signs = quant.get_signs(torch.device("cuda"))
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16, generator=g)
    quant.reset_stats(0)
    first = quant.dual(x, signs)
    again = quant.dual(x.reshape(-1, 384), signs)           # a new view of the same storage
    assert again[0].data is first[0].data and again[1].data is first[1].data
    assert quant.stats()["activation_pack_reused"] == 1 and quant.stats()["quant"] == 4
    x.mul_(2)                                                # version bump
    fresh = quant.dual(x, signs)
    assert fresh[0].data is not first[0].data and quant.stats()["activation_pack_reused"] == 1
    assert not torch.equal(fresh[0].pts, first[0].pts)
    other = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16, generator=g)
    assert quant.dual(other, signs)[0].data is not fresh[0].data
    back = quant.dual(x, signs)                              # only the last pair is remembered
    assert back[0].data is not fresh[0].data and torch.equal(back[0].data, fresh[0].data)
    assert torch.equal(back[1].data, fresh[1].data) and torch.equal(back[0].scale, fresh[0].scale)
    a, b = quant.dual(x, signs, sr=True), quant.dual(x, signs, sr=True)
    assert a[0].data is not b[0].data and not torch.equal(a[0].data, b[0].data)


@pytest.mark.parametrize("profile", ["balanced", "short128", "conservative", "same_as_v5", "experimental_m4v4"])
def test_optimizer_emitted_packings_leave_captured_training_unchanged(profile):
    """prepack: the update kernel also writes the next forward's weight packings (one cooperative launch per weight).  The
    packings are byte-identical to what the forward would compute, so weights and optimizer state after captured steps are
    the same with and without it, and the forward of the captured step holds no weight quantiser any more."""
    import nvfp4_training as nv
    from nvfp4_training._runtime import load_runtime
    rng = load_runtime()[2]
    x, y = batch(256, seed=3)
    results = []
    for prepack in (False, True):
        rng.reset_stats(5)
        model = nv.enable_nvfp4(make_model(seed=4).cuda(), profile=profile, lr=1e-3)
        opt = model.nvfp4_optimizer
        opt.param_groups[0]["prepack"] = prepack
        nv.train_step(model, mse, x, y)
        with nv.capture_step(model, mse, x, y, steps=4) as graph:
            seen = rng.stats()
            losses = [graph.step(x, y).item() for _ in range(4)]
        nv.check_finite(model)
        assert not any(hasattr(p, "_v6_pack") for p in model.parameters())      # the capture took its buffers with it
        if prepack:
            assert seen.get("prepacked_weight", 0) == 3 and getattr(opt, "prepacked", 0) == 3
        nv.train_step(model, mse, x, y)      # eager training continues on the ordinary path
        results.append((losses, state_bytes(model)))
    assert results[0][0] == results[1][0]
    assert same(results[0][1], results[1][1])


def test_prepack_is_refused_where_the_reference_refuses_it():
    from nvfp4_training._backend.engine import configure
    with pytest.raises(ValueError, match="one weight encoding strategy"):
        configure(make_model(), "fp4", "half16_v8", prepack=True, remat=True, direct=True)
    with pytest.raises(ValueError, match="FP8 storage"):
        configure(make_model(), "fp4", "float8_m4v4_sqrt", prepack=True, direct=True)


@pytest.mark.parametrize("fmt", ["split24_m4", "sr16_m4", "sr16_m4v4", "float8_v8"])
def test_storage_formats_outside_the_profiles_train(fmt):
    """The four entries of the reference's FORMATS table that no public profile selects (engine6.py:13-17): configure
    accepts them, the model trains, state tensors have the reference's dtypes and sizes."""
    from nvfp4_training._backend.engine import configure
    from nvfp4_training._backend.optimizer import FORMATS
    import nvfp4_training as nv
    master, vb, mb = FORMATS[fmt]
    from nvfp4_training._backend.linear import AutocastLinear, Linear6
    model, opt = configure(make_model().cuda(), "fp4", fmt, lr=1e-3)
    for module in model.modules():          # what prepare_training does after configure: layers run in BF16 under autocast
        if isinstance(module, Linear6):
            module.__class__ = AutocastLinear
    model.nvfp4_optimizer = opt
    x, y = batch(256)
    losses = []
    for _ in range(12):
        losses.append(nv.train_step(model, mse, x, y).item())
    nv.check_finite(model)
    assert losses[-1] < losses[0]
    w = model[3].weight
    want = {24: torch.bfloat16, 16: torch.bfloat16, 8: torch.float8_e4m3fn}[master]
    state = opt.state[w]
    assert w.dtype == want and ("tail" in state) == (master == 24)
    n = w.numel()
    assert state["m"].numel() == ((n + 1) // 2 if mb == 4 and vb != 4 else n)
    assert ("v" in state) == (vb != 4 or mb != 4)
