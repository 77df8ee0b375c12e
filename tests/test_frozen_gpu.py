"""Frozen NVFP4 storage on the GPU: parity with the trainable NVFP4 layer, cache save / load, pointwise and attention
wrappers, graph replay with a device SR seed.  Cases follow the reference's tests/test_frozen.py:47-136."""
import copy

import pytest
import torch
from torch import nn
from torch.nn import functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture()
def backend():
    from nvfp4_training import frozen
    torch.manual_seed(123)
    return frozen.runtime()[0]


class Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.input = nn.Linear(128, 128)
        self.frozen = nn.Linear(128, 128).requires_grad_(False)
        self.output = nn.Linear(128, 4)

    def forward(self, x):
        x = self.input(x)
        for _ in range(2):
            x = x + 0.1 * self.frozen(x)
        return self.output(x)


@pytest.mark.parametrize("k,n", [(128, 256), (65, 67), (384, 129)])
def test_native_parity_and_cache(backend, tmp_path, k, n):
    from nvfp4_training import pack_frozen_layers, save_frozen_cache, load_frozen_cache, frozen
    from nvfp4_training._runtime import load_runtime
    original = nn.Linear(k, n, device="cuda", dtype=torch.bfloat16).requires_grad_(False)
    model = pack_frozen_layers(copy.deepcopy(original), include=("*",))
    native = load_runtime()[3]
    reference = copy.deepcopy(original)
    reference.__class__ = native
    reference.register_buffer("_nvfp4_signs", backend.get_signs(original.weight.device), persistent=False)
    reference._nvfp4_save_packed = True
    reference.weight._v6_remat = True
    x = torch.randn(17, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(17, n, device="cuda", dtype=torch.bfloat16)
    backend._SEED = 123
    a = reference(x)
    ga = torch.autograd.grad(a, x, g)[0]
    backend._SEED = 123
    b = model(x)
    gb = torch.autograd.grad(b, x, g)[0]
    assert torch.equal(a, b) and torch.equal(ga, gb)
    # and both equal the dense product to FP4 accuracy
    dense = F.linear(x.float(), original.weight.float(), original.bias.float())
    assert ((b.float() - dense).norm() / dense.norm()).item() < 0.15
    inv = frozen.inventory(model)
    assert inv["master_parameter_elements"] == 0 and inv["projections"] == 1 and inv["source_elements"] == k * n
    path = tmp_path / "cache.pt"
    info = save_frozen_cache(path, model, model_fingerprint="synthetic-v1")
    assert info["projections"] == 1 and len(info["sha256"]) == 64
    count = frozen.PACKS
    restored = load_frozen_cache(path, copy.deepcopy(original), expected_fingerprint="synthetic-v1")
    assert frozen.PACKS == count, "a cache load must not quantise"
    assert torch.equal(model(x), restored(x))
    with pytest.raises(ValueError):
        load_frozen_cache(path, copy.deepcopy(original), expected_fingerprint="wrong-revision")
    with path.open("ab") as f:
        f.write(b"changed")
    with pytest.raises(ValueError, match="checksum"):
        load_frozen_cache(path, copy.deepcopy(original), expected_fingerprint="synthetic-v1")


def test_pointwise_and_attention_cache(backend, tmp_path):
    from nvfp4_training import pack_frozen_layers, save_frozen_cache, load_frozen_cache
    modules = [nn.Conv2d(16, 32, 1).cuda().bfloat16(), nn.MultiheadAttention(128, 4, batch_first=True).cuda().bfloat16()]
    for i, original in enumerate(modules):
        original.requires_grad_(False)
        model = pack_frozen_layers(copy.deepcopy(original), include=("*",))
        conv = isinstance(original, nn.Conv2d)
        x = (torch.randn(2, 16, 3, 3, device="cuda", dtype=torch.bfloat16) if conv
             else torch.randn(2, 9, 128, device="cuda", dtype=torch.bfloat16))

        def call(m):
            return m(x) if conv else m(x, x, x, need_weights=False)[0]
        dense, packed = call(original).float(), call(model).float()
        assert ((packed - dense).norm() / dense.norm()).item() < (0.15 if conv else 0.35)   # two FP4 layers around the softmax
        path = tmp_path / f"cache{i}.pt"
        save_frozen_cache(path, model, model_fingerprint="synthetic-v1")
        restored = load_frozen_cache(path, copy.deepcopy(original), expected_fingerprint="synthetic-v1")
        assert torch.equal(call(model), call(restored))
    with pytest.raises(ValueError, match="self attention"):
        model(x, x, x)


def test_graph_backward_dynamic_sr_and_changed_input(backend):
    from nvfp4_training import pack_frozen_layers, capture_frozen
    model = pack_frozen_layers(Toy().cuda(), include=("frozen",), keep=("input", "output"))
    x = torch.randn(8, 128, device="cuda")
    target = torch.randn(8, 4, device="cuda")

    def objective(m, x, y):
        return F.mse_loss(m(x).float(), y)
    backend._SEED = 0
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = objective(model, x, target)
    loss.backward()
    trainable = [p for p in model.parameters() if p.requires_grad]
    expected = [p.grad.detach().clone() for p in trainable]
    del loss
    with capture_frozen(model, objective, x, target) as replay:
        assert replay.sr_calls == 2
        value = replay.replay(x, target).clone()
        torch.cuda.synchronize()
        grads = [p.grad.detach().clone() for p in trainable]
        for a, b in zip(expected, grads):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
        replay.replay(x, target)
        torch.cuda.synchronize()
        assert any(not torch.equal(a, p.grad) for a, p in zip(grads, trainable)), "SR noise must change between replays"
        changed = replay.replay(x + 0.25, target).clone()
        torch.cuda.synchronize()
        assert not torch.equal(value, changed)
        with pytest.raises(ValueError):
            replay.replay(x[:1], target[:1])
        model.frozen.data = model.frozen.data.clone()
        with pytest.raises(RuntimeError, match="packed buffers"):
            replay.replay(x, target)
    with pytest.raises(RuntimeError, match="closed"):
        replay.replay(x, target)


def test_inference_graph(backend):
    from nvfp4_training import pack_frozen_layers, capture_frozen
    model = pack_frozen_layers(nn.Linear(128, 64).cuda().requires_grad_(False), include=("*",))
    x = torch.randn(8, 128, device="cuda")
    with torch.no_grad():
        expected = model(x)
    with capture_frozen(model, lambda m, x: m(x), x, backward=False) as replay:
        actual = replay.replay(x).clone()
        torch.cuda.synchronize()
        assert torch.equal(actual, expected)
        assert replay.sr_calls == 0


def test_input_gradient_replay(backend):
    from nvfp4_training import pack_frozen_layers, capture_frozen
    model = pack_frozen_layers(nn.Linear(128, 64).cuda().requires_grad_(False), include=("*",))
    x = torch.randn(8, 128, device="cuda", requires_grad=True)

    def objective(m, x):
        return m(x).float().square().mean()
    backend._SEED = 0
    expected = torch.autograd.grad(objective(model, x), x)[0]
    with capture_frozen(model, objective, x) as replay:
        replay.replay(x)
        torch.cuda.synchronize()
        assert torch.equal(expected, replay.inputs[0].grad)
        assert x.grad is None   # graphs outside the replay are not captured
