"""GPU parity of the fused compressed-AdamW kernel: against golden vectors produced by the reference's own Triton
kernels, and against the CPU oracle on larger / ragged tensors.  Bit exact, through the C ABI."""
import numpy as np
import pytest
import torch

import oracle as O
from conftest import GOLDEN

pytestmark = pytest.mark.gpu

FORMATS = ["half16_v8", "half16_v8b128", "split24_v8", "tile32", "sr16_v8", "half16_m4v4_sqrt", "float8_m4v4_sqrt", "half16_m8v4",
           "split24_m4", "sr16_m4", "sr16_m4v4", "float8_v8"]
TORCH_OF = {32: torch.float32, 24: torch.bfloat16, 17: torch.float16, 16: torch.bfloat16, 8: torch.uint8}


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLDEN / "adamw_reference.npz")


def _dev(a, view=None):
    t = torch.from_numpy(a.copy()).cuda()
    return t


def _state(n, fmt):
    master, vb, mb = O.FORMATS[fmt]
    width = O.state_block(fmt)
    m = torch.zeros((n + 1) // 2 if mb == 4 and vb != 4 else n, dtype=torch.uint8 if mb == 4 else torch.int8, device="cuda")
    ms = torch.zeros(-(-n // (64 if mb == 4 else width)), dtype=torch.float32, device="cuda")
    vs = torch.zeros(-(-n // (64 if vb == 4 else width)), dtype=torch.float32, device="cuda")
    v = None
    if vb != 4 or mb != 4:
        v = torch.zeros(-(-n // 2) if vb == 4 else n, dtype=torch.uint8 if vb < 16 else torch.float16, device="cuda")
    return m, v, ms, vs


def _np(t):
    if t is None:
        return None
    t = t.detach().cpu()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def _hyper32(h):
    return {k: float(np.float32(v)) for k, v in h.items()}


@pytest.mark.parametrize("fmt", FORMATS)
def test_update_matches_reference_golden(native, gold, fmt):
    master, vb, mb = O.FORMATS[fmt]
    rows, cols, stride = (int(x) for x in gold["meta"])
    n = rows * cols
    lr, b1, b2, eps, wd = (float(x) for x in gold["hyper"])
    p0 = gold[f"{fmt}_p0"]
    p = torch.from_numpy(p0.copy()).cuda()
    if master in (24, 17, 16):
        p = p.view(torch.int16).view(TORCH_OF[master])
    tail = torch.from_numpy(gold[f"{fmt}_tail0"].copy()).cuda() if master == 24 else None
    unit = torch.from_numpy(gold[f"{fmt}_unit0"].copy()).cuda() if master == 8 else None
    m, v, ms, vs = _state(n, fmt)
    sa, sb = (torch.tensor([float(x)], device="cuda") for x in gold["scales"])
    extra = torch.from_numpy(gold["extra"].copy()).cuda()
    scale = torch.zeros(1, device="cuda")
    for t in (1, 2, 3):
        packed = t < 3
        grad = torch.from_numpy((gold[f"raw{t - 1}"] if packed else gold["dense"]).copy()).cuda()
        if packed:
            grad = grad.view(torch.int16).view(torch.bfloat16)
        native.adamw_step(p, master, grad, m, v, ms, vs, vbits=vb, mbits=mb, nonlinear_m=fmt.endswith("_sqrt"),
                          state_block=O.state_block(fmt), hyper=O.adam_hyper(lr, (b1, b2), eps, wd, t), step=t, key=12345 + 7919 * 3,
                          grad_kind=2 if packed else 0, grad_cols=cols, grad_stride=stride, sa=sa, sb=sb,
                          extra=extra if t == 2 else None, tail=tail, unit=unit, scale_out=scale)
        got = dict(p=_np(p), m=_np(m), v=_np(v), ms=_np(ms), vs=_np(vs), tail=_np(tail), unit=_np(unit), scale=_np(scale))
        for name, val in got.items():
            if val is None:
                continue
            want = gold[f"{fmt}_s{t}_{name}"]
            assert np.array_equal(val.view(np.uint8), want.view(np.uint8)), f"{fmt} step {t} {name}: {(val != want).sum()} differ"


@pytest.mark.parametrize("fmt", ["half16_v8", "half16_v8b128", "split24_v8", "tile32", "half16_m4v4_sqrt", "float8_m4v4_sqrt"])
@pytest.mark.parametrize("n", [4096, 100003, 1 << 20])
def test_update_matches_oracle_on_ragged_sizes(native, fmt, n):
    master, vb, mb = O.FORMATS[fmt]
    g = torch.Generator().manual_seed(n)
    w = torch.randn(n, generator=g) * 0.02
    w[::101] *= 1e-3
    tail = unit = None
    if master == 32:
        p = w.clone().cuda()
    elif master == 8:
        u0 = 2.0 ** np.ceil(np.log2(max(float(w.abs().max()), 1e-20) / 48.0))
        unit = torch.full((-(-n // 512),), u0, dtype=torch.float32, device="cuda")
        p = (w / u0).to(torch.float8_e4m3fn).view(torch.uint8).cuda()
    else:
        p, tail = native.split_init(w.cuda(), master)
        hi, tl = O.split_init(w.numpy(), master)
        assert np.array_equal(_np(p), hi) and (tl is None or np.array_equal(_np(tail), tl))
    m, v, ms, vs = _state(n, fmt)
    op, om, ov, oms, ovs = (None if x is None else _np(x).copy() for x in (p, m, v, ms, vs))
    otail = None if tail is None else _np(tail).copy()
    ounit = None if unit is None else _np(unit).copy()
    scale = torch.zeros(1, device="cuda")
    for t in (1, 2):
        grad = (torch.randn(n, generator=g) * (3e-3 if t == 1 else 50.0)).bfloat16()
        # state blocks whose scale leaves the range of the shared-reciprocal division (all-zero gradients: scale 1e-30;
        # gradients near 1e-14: scale about 1e-17) and one far up the range
        grad[:1024] = 0
        grad[1024:2048] *= 1e-12
        grad[2048:2560] *= 1e12
        h = O.adam_hyper(3e-4, (0.9, 0.95), 1e-8, 0.1, t)
        native.adamw_step(p, master, grad.cuda(), m, v, ms, vs, vbits=vb, mbits=mb, nonlinear_m=fmt.endswith("_sqrt"),
                          state_block=O.state_block(fmt), hyper=h, step=t, key=777, tail=tail, unit=unit, scale_out=scale)
        part = O.adam_update(fmt, op, _np(grad), om, ov, oms, ovs, step=t, key=777, hyper=h, tail=otail, unit=ounit, grad_kind=1)
        for name, got, want in (("p", p, op), ("m", m, om), ("v", v, ov), ("ms", ms, oms), ("vs", vs, ovs), ("tail", tail, otail), ("unit", unit, ounit)):
            if got is None:
                continue
            assert np.array_equal(_np(got).view(np.uint8), want.view(np.uint8)), f"{fmt} n={n} step {t} {name}"
        assert np.float32(scale.item()) == O.finish_scale(part)


def test_plain_small_tensor_path(native, gold):
    lr, b1, b2, eps, wd = (float(x) for x in gold["hyper"])
    p, g = (torch.from_numpy(gold[k].copy()).cuda() for k in ("plain_p0", "plain_g"))
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for t in (1, 2):
        native.adamw_plain(p, g, m, v, hyper=O.adam_hyper(lr, (b1, b2), eps, wd, t))
        for name, got in (("p", p), ("m", m), ("v", v)):
            assert np.array_equal(_np(got).view(np.uint32), gold[f"plain_s{t}_{name}"].view(np.uint32)), (t, name)


def test_device_control_tensor_overrides_step_scalars(native):
    n = 8192
    g = torch.Generator().manual_seed(1)
    w = (torch.randn(n, generator=g) * 0.02).cuda()
    grad = torch.randn(n, generator=g).bfloat16().cuda()
    outs = []
    for use_ctrl in (False, True):
        p, _ = native.split_init(w, 17)
        m, v, ms, vs = _state(n, "half16_v8")
        h = O.adam_hyper(1e-3, (0.9, 0.999), 1e-8, 0.01, 5)
        ctrl = None
        hh, step = dict(h), 5
        if use_ctrl:
            ctrl = torch.tensor([h["c1"], h["c2"], 0.0, 0.0], dtype=torch.float32, device="cuda")
            ctrl[3:4].view(torch.int32)[0] = 5
            hh.update(c1=123.0, c2=456.0)
            step = 99
        native.adamw_step(p, 17, grad, m, v, ms, vs, vbits=8, mbits=8, nonlinear_m=False, state_block=512, hyper=hh, step=step,
                          key=4242, ctrl=ctrl)
        outs.append((p.clone(), m.clone(), v.clone()))
    assert all(torch.equal(a, b) for a, b in zip(*outs))


def test_scale_reduction_is_independent_of_earlier_amax_calls(native):
    """The quantiser's amax pass and the optimizer's amax reduction share one scratch block; they must not see each
    other's leftovers."""
    n = 65536
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(n, generator=g) * 0.02).cuda()
    grad = torch.randn(n, generator=g).bfloat16().cuda()
    native.amax(torch.randn(512, 512, device="cuda").bfloat16())     # leaves partial maxima behind
    p, _ = native.split_init(w, 17)
    m, v, ms, vs = _state(n, "half16_v8")
    scale = torch.full((1,), -1.0, device="cuda")
    h = O.adam_hyper(1e-3, (0.9, 0.999), 1e-8, 0.01, 1)
    native.adamw_step(p, 17, grad, m, v, ms, vs, vbits=8, mbits=8, nonlinear_m=False, state_block=512, hyper=h, step=1, key=9,
                      scale_out=scale)
    want = native.amax(p.view(1, -1))[1]
    assert scale.item() == want.item()
    native.adamw_step(p, 17, grad, m, v, ms, vs, vbits=8, mbits=8, nonlinear_m=False, state_block=512, hyper=h, step=2, key=9,
                      scale_out=scale)
    assert scale.item() == native.amax(p.view(1, -1))[1].item()


@pytest.mark.parametrize("fmt", ["half16_v8", "half16_v8b128", "split24_v8", "tile32", "half16_m4v4_sqrt"])
@pytest.mark.parametrize("rows,cols", [(256, 512), (130, 200), (1024, 3072)])
def test_update_with_emitted_packings_equals_update_then_quantise(native, fmt, rows, cols):
    """nvfp4_adamw_step_prepack: same master / moments / scale as nvfp4_adamw_step, and packings byte-identical to the pair
    quantiser run on the updated weight with the new scale (two updates in a row: the grid barrier word resets itself)."""
    from _util import signs_dev
    master, vb, mb = O.FORMATS[fmt]
    n = rows * cols
    g = torch.Generator().manual_seed(rows + cols)
    w = (torch.randn(rows, cols, generator=g) * 0.02).cuda()
    states = []
    for _ in range(2):
        if master == 32:
            p, tail = w.clone(), None
        else:
            p, tail = native.split_init(w, master)
        states.append((p, tail, *_state(n, fmt)))
    (pa, ta, ma, va, msa, vsa), (pb, tb, mb_, vb_, msb, vsb) = states
    sa_, sb_ = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    mp, kp = native.round128(rows), native.round128(cols)
    pack = (torch.zeros((mp, kp // 2), dtype=torch.uint8, device="cuda"), torch.zeros((mp // 128 * 32, kp // 64 * 16), dtype=torch.uint8, device="cuda"),
            torch.zeros((kp, mp // 2), dtype=torch.uint8, device="cuda"), torch.zeros((kp // 128 * 32, mp // 64 * 16), dtype=torch.uint8, device="cuda"))
    for t in (1, 2):
        grad = (torch.randn(rows, cols, generator=g) * 3e-3).bfloat16().cuda()
        h = O.adam_hyper(3e-4, (0.9, 0.95), 1e-8, 0.1, t)
        common = dict(vbits=vb, mbits=mb, nonlinear_m=fmt.endswith("_sqrt"), state_block=O.state_block(fmt), hyper=h, step=t, key=4242)
        native.adamw_step(pa.view(-1), master, grad.view(-1), ma, va, msa, vsa, tail=None if ta is None else ta.view(-1), scale_out=sa_, **common)
        native.adamw_step_prepack(pb, master, grad, mb_, vb_, msb, vsb, pack=pack, tail=tb, scale_out=sb_, **common)
        native.check_status()
        for got, want in ((pb, pa), (mb_, ma), (vb_, va), (msb, msa), (vsb, vsa), (tb, ta), (sb_, sa_)):
            if want is not None:
                assert torch.equal(got.view(torch.uint8).flatten(), want.view(torch.uint8).flatten())
        d, s, _, dt, st = native.quantize(pa, signs_dev(), mp, kp, 0, False, 0, given_scale=sa_.reshape(()), pair=True)
        for got, want, name in zip(pack, (d, s, dt, st), ("payload", "scales", "payload^T", "scales^T")):
            assert torch.equal(got, want), f"{fmt} {rows}x{cols} step {t}: {name}"
