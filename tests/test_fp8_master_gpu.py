"""FP8 master weights (profile experimental_fp8_master) on the GPU: the weight quantiser that reads E4M3 codes and their
per-512 units directly, unit growth in the update kernel, and the range / checkpoint behaviour the reference tests in
tests/test_fp8_master_range.py.  Fixtures come from the reference's own Triton kernels (tests/golden/make_golden_fp8.py)."""
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch
from torch import nn

import oracle as O
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN / "fp8_master_reference.npz")


@pytest.mark.parametrize("case", ["grown", "random_units"])
def test_fp8_weight_quantiser_matches_reference(native, gold, case):
    """master8.encode: both NVFP4 orientations from the stored codes, bit for bit; ragged 65 x 67 and 130 x 96 weights."""
    g = gold
    keys = ("s2_p", "s2_unit", "enc_scale", "enc_d", "enc_s", "enc_dt", "enc_st") if case == "grown" else \
           ("b_p", "b_unit", "b_scale", "b_d", "b_s", "b_dt", "b_st")
    p, unit, scale = (torch.from_numpy(g[k].copy()).cuda() for k in keys[:3])
    d, s, dt, st = native.quantize_fp8_weight(p, unit, scale)
    for got, key in ((d, keys[3]), (s, keys[4]), (dt, keys[5]), (st, keys[6])):
        assert np.array_equal(got.cpu().numpy(), g[key]), key
    # single orientations (the recompute-in-backward mode) give the same bytes
    d1, s1, _, _ = native.quantize_fp8_weight(p, unit, scale, col=False)
    _, _, dt1, st1 = native.quantize_fp8_weight(p, unit, scale, row=False)
    assert torch.equal(d1, d) and torch.equal(s1, s) and torch.equal(dt1, dt) and torch.equal(st1, st)


def test_fp8_unit_growth_matches_reference(native, gold):
    """adam_kernel.update with an update beyond 448 x unit: exactly the first and the last unit grow, the other blocks keep
    every byte; then an ordinary step on the grown units."""
    g = gold
    lr, b1, b2, eps, wd = (float(x) for x in g["hyper"])
    p = torch.from_numpy(g["p0"].reshape(-1).copy()).cuda()
    unit = torch.from_numpy(g["unit0"].copy()).cuda()
    n = p.numel()
    m = torch.zeros(n, dtype=torch.uint8, device="cuda")
    ms, vs = (torch.zeros(-(-n // 64), dtype=torch.float32, device="cuda") for _ in range(2))
    scale = torch.zeros(1, device="cuda")
    for t in (1, 2):
        grad = torch.from_numpy(g["grads"][t - 1].copy()).cuda()
        native.adamw_step(p, 8, grad, m, None, ms, vs, vbits=4, mbits=4, nonlinear_m=True, state_block=512,
                          hyper=O.adam_hyper(lr, (b1, b2), eps, wd, t), step=t, key=int(g["key"][0]), unit=unit, scale_out=scale)
        for name, got in (("p", p), ("unit", unit), ("m", m), ("ms", ms), ("vs", vs)):
            want = g[f"s{t}_{name}"].reshape(-1)
            assert np.array_equal(got.cpu().numpy().view(np.uint8), want.view(np.uint8)), f"step {t} {name}"
        assert np.float32(scale.item()) == O.finish_scale(g[f"s{t}_part"])


def _model():
    import nvfp4_training as nv
    layer = nn.Linear(65, 67, bias=False)
    with torch.no_grad():
        layer.weight.fill_(0.0001)
    return nv.prepare_training(layer.cuda(), profile="experimental_fp8_master", precision="fp4", lr=.25, betas=(0., 0.), eps=1e-8,
                               weight_decay=0.)


def test_fp8_master_range_checkpoint_and_nonfinite_detection(native):
    """The reference's tests/test_fp8_master_range.py:17-60 on this backend."""
    import nvfp4_training as nv
    from nvfp4_training._backend.linear import decoded, encode
    from nvfp4_training._backend.quant import pair
    layer, opt = _model()
    p = layer.weight
    initial = p.detach().view(torch.uint8).clone()
    units = p._v6_unit.clone()
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "state.pt"
        nv.save_checkpoint(path, layer)
        legacy = torch.load(path, map_location="cpu", weights_only=True)
        legacy["model"]["_v6_unit_buffer"] = legacy["model"]["_v6_unit_buffer"][0].clone()   # the old scalar-unit layout
        torch.save(legacy, path)
        other, _ = _model()
        assert nv.load_checkpoint(path, other) == 0
        assert torch.equal(other.weight._v6_unit, units)
        assert torch.equal(decoded(other.weight), decoded(p))
        grad = torch.zeros(p.shape, device="cuda")
        grad.flatten()[1] = 1.
        grad.flatten()[-1] = -1.
        p.grad = grad.to(p.dtype)
        opt.step()
        nv.check_finite(layer)
        vals = decoded(p).reshape(-1).float()
        assert .22 < -vals[1].item() < .29 and .22 < vals[-1].item() < .29
        assert (p._v6_unit > units).nonzero().flatten().tolist() == [0, len(units) - 1]
        assert torch.equal(initial.flatten()[512:-512], p.view(torch.uint8).flatten()[512:-512])
        assert p._v6_unit[0] > units[0] and .22 > 448 * units[0].item()
        plain = (p.float().flatten() * p._v6_unit.repeat_interleave(512)[:p.numel()]).reshape(p.shape).bfloat16()
        assert torch.equal(decoded(p), plain)
        scale = plain.float().abs().max() / 2688
        encoded = encode(p, scale)
        reference = pair(plain, scale)
        for left, right in zip(encoded, reference):
            assert torch.equal(left, right)
        nv.save_checkpoint(path, layer)
        assert nv.load_checkpoint(path, other) == 1
        assert torch.equal(decoded(other.weight), plain)
        assert torch.equal(p._v6_unit, other.weight._v6_unit)
        p.grad.view(torch.uint8).flatten()[1] = 127      # a NaN code in the gradient
        opt.step()
        with pytest.raises(FloatingPointError):
            nv.check_finite(layer)
