"""GPU parity of the sm_100a quantiser against the CPU oracle and the reference-generated goldens.
Every call goes through the C ABI (ctypes), bit exact."""
import numpy as np
import pytest
import torch

import oracle as O
from _util import alloc_packing, outlier_tensor, signs_dev, to_oracle

pytestmark = pytest.mark.gpu

MODES = {"rne": (0, O.RNE), "hash": (2, O.SR_HASH), "philox": (4, O.SR_PHILOX)}
SHAPES = [(128, 256), (40, 70), (193, 129), (17, 35), (11, 19), (256, 128), (1, 1), (129, 16)]


def _cmp(got_packed, got_scales, want):
    gp, gs = got_packed.cpu().numpy(), got_scales.cpu().numpy()
    assert np.array_equal(gs, want[1]), f"scales differ in {(gs != want[1]).sum()} bytes"
    assert np.array_equal(gp, want[0]), f"payload differs in {(gp != want[0]).sum()} bytes"


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("rht", [False, True])
def test_quantize_operator_matches_oracle(native, shape, dtype, mode, rht):
    x = outlier_tensor(shape, seed=shape[0] * 1000 + shape[1], dtype=dtype)
    xd = x.cuda()
    flag, omode = MODES[mode]
    signs = signs_dev()
    mp, kp = native.round128(shape[0]), native.round128(shape[1])
    packed, scales, pts = native.quantize(xd, signs, mp, kp, flag, rht, 173)
    xo, kind = to_oracle(x)
    want = O.quantize(xo, sr_mode=omode, rht=rht, seed=173, kind=kind)
    assert np.float32(pts.item()) == want[2]
    _cmp(packed, scales, want)


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("rht", [False, True])
def test_transposed_and_strided_views(native, mode, rht):
    flag, omode = MODES[mode]
    signs = signs_dev()
    base = outlier_tensor((193, 129), seed=5, dtype=torch.bfloat16)
    for view_of in (lambda t: t.t(), lambda t: t[::2, ::2], lambda t: t[3:, 5:], lambda t: t.t()[::3]):
        x = view_of(base)
        xd = view_of(base.cuda())
        mp, kp = native.round128(x.shape[0]), native.round128(x.shape[1])
        packed, scales, pts = native.quantize(xd, signs, mp, kp, flag, rht, 7)
        xo, kind = to_oracle(x)
        want = O.quantize(xo, sr_mode=omode, rht=rht, seed=7, kind=kind)
        assert np.float32(pts.item()) == want[2]
        _cmp(packed, scales, want)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d", "e", "f"])
def test_dual_matches_reference_golden(native, golden_quant, tag):
    g = golden_quant
    sr, seed, is_bf16 = (int(v) for v in g[f"dual_{tag}_meta"])
    raw = g[f"dual_{tag}_x"]
    x = (torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16) if is_bf16 else torch.from_numpy(raw)).cuda()
    m, n = x.shape
    mp, np_ = native.round128(m), native.round128(n)
    signs = torch.from_numpy(g["signs"]).cuda()
    a4 = native.amax(x)
    rp, rs = alloc_packing(mp, np_)
    cp, cs = alloc_packing(np_, mp)
    flags = 2 if sr else 0
    native.quantize_tile(x, signs,
                         row=dict(packed=rp, scales=rs, pts=a4[1:2], flags=flags, seed=seed),
                         col=dict(packed=cp, scales=cs, pts=a4[2:3], flags=flags | 1, seed=seed + 1))
    assert np.float32(a4[1].item()) == g[f"dual_{tag}_row_pts"][0]
    assert np.float32(a4[2].item()) == g[f"dual_{tag}_col_pts"][0]
    _cmp(rp, rs, (g[f"dual_{tag}_row_data"], g[f"dual_{tag}_row_scale"]))
    _cmp(cp, cs, (g[f"dual_{tag}_col_data"], g[f"dual_{tag}_col_scale"]))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_weight_pair_matches_reference_golden(native, golden_quant, tag):
    g = golden_quant
    kind = int(g[f"pair_{tag}_kind"][0])
    raw = g[f"pair_{tag}_w"]
    if kind == 0:
        w = torch.from_numpy(raw)
    else:
        w = torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16 if kind == 1 else torch.float16)
    w = w.cuda()
    pts = torch.from_numpy(g[f"pair_{tag}_pts"]).cuda()
    mp, kp = native.round128(w.shape[0]), native.round128(w.shape[1])
    d, s, p, dt, st = native.quantize(w, signs_dev(), mp, kp, 0, False, 0, given_scale=pts, pair=True)
    _cmp(d, s, (g[f"pair_{tag}_data"], g[f"pair_{tag}_scale"]))
    _cmp(dt, st, (g[f"pair_{tag}_data_t"], g[f"pair_{tag}_scale_t"]))
    # the amax kernel reproduces the scale the optimizer would cache
    a4 = native.amax(w)
    assert np.float32(a4[1].item()) == g[f"pair_{tag}_pts"][0]


def test_device_seed_base_shifts_the_seed(native):
    x = outlier_tensor((128, 128), seed=3).cuda()
    signs = signs_dev()
    base = torch.tensor([41], dtype=torch.int32, device="cuda")
    a = native.quantize(x, signs, 128, 128, 2, True, 100, seed_base=base)
    b = native.quantize(x, signs, 128, 128, 2, True, 141)
    c = native.quantize(x, signs, 128, 128, 2, True, 100)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert not torch.equal(a[0], c[0])


@pytest.mark.parametrize("hi_first", [False, True])
def test_hi_first_nibble_order_and_dequantize(native, hi_first):
    x = outlier_tensor((130, 77), seed=8, dtype=torch.float32)
    xd = x.cuda()
    signs = signs_dev()
    a4 = native.amax(xd)
    rp, rs = alloc_packing(256, 128)
    native.quantize_tile(xd, signs, row=dict(packed=rp, scales=rs, pts=a4[1:2], flags=8 if hi_first else 0, seed=0))
    want = O.quantize(x.numpy(), hi_first=hi_first)
    _cmp(rp, rs, want)
    for dtype in (torch.float32, torch.bfloat16):
        got = native.dequantize(rp, rs, a4[1:2], 130, 77, hi_first=hi_first, dtype=dtype).float().cpu().numpy()
        ref = O.dequantize(want[0], want[1], want[2], 130, 77, hi_first=hi_first)
        if dtype == torch.bfloat16:
            ref = O.from_bf16_bits(O.to_bf16_bits(ref))
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_padding_is_written_and_zero_stays_zero(native):
    x = torch.zeros((17, 35), dtype=torch.bfloat16, device="cuda")
    for flag in (0, 2, 4):
        for rht in (False, True):
            p, s, t = native.quantize(x, signs_dev(), 128, 128, flag, rht, 1)
            assert not p.any().item() and (s == 0x08).all().item()


def test_error_codes_become_python_exceptions(native):
    x = torch.zeros((16, 16), dtype=torch.float64, device="cuda")
    with pytest.raises(TypeError):
        native.quantize(x, signs_dev(), 128, 128, 0, False, 0)
    y = torch.zeros((16, 16), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        native.quantize(y, signs_dev(), 256, 128, 0, False, 0)


def test_full_size_config_matches_oracle_and_round_trips(native):
    """4096 x 4096 BF16 with 0.1 % x50 outliers, RNE and SR seed 0, with and without the H16 RHT."""
    x = outlier_tensor((4096, 4096), seed=0)
    xd = x.cuda()
    xo, _ = to_oracle(x)
    signs0 = torch.from_numpy(O.default_signs(0)).cuda()
    for flag, omode in ((0, O.RNE), (2, O.SR_HASH), (4, O.SR_PHILOX)):
        for rht in (False, True):
            p, s, t = native.quantize(xd, signs0, 4096, 4096, flag, rht, 0)
            want = O.quantize(xo, sr_mode=omode, rht=rht, seed=0, signs=O.default_signs(0))
            assert np.float32(t.item()) == want[2]
            _cmp(p, s, want)
            if not rht:
                back = native.dequantize(p, s, t, 4096, 4096).cpu()
                rel = (back - x.float()).norm() / x.float().norm()
                assert rel < 0.15


def _cuda_quant_names():
    from conftest import GOLDEN
    return [str(n) for n in np.load(GOLDEN / "cuda_quant_reference.npz")["names"]]


@pytest.mark.parametrize("name", _cuda_quant_names())
def test_quantize_matches_reference_cuda_kernels(native, golden_cuda_quant, name):
    """The `quantize` operator against outputs of the reference's own CUDA kernels (run on the host by
    tests/golden/make_golden_cuda_quant.py): rows, transposed and strided views, SR x RHT, BF16 and FP32 sources."""
    from conftest import cuda_quant_case
    g = golden_cuda_quant
    x, sr, rht, seed, given, want = cuda_quant_case(g, name)
    kind = int(g[f"{name}_meta"][0])
    base = (x.t() if kind == 1 else x).cuda() if kind != 2 else None
    if kind == 2:
        raw = g["base_" + str(g[f"{name}_base"])]
        is_bf16 = int(g[f"{name}_meta"][1])
        full = torch.from_numpy(raw.view(np.int16)).view(torch.bfloat16) if is_bf16 else torch.from_numpy(raw)
        xd = full.cuda()[::2, ::2]
    else:
        xd = base.t() if kind == 1 else base
    assert xd.stride() == x.stride()
    signs = torch.from_numpy(g["signs"]).cuda()
    scale = None if given is None else torch.tensor(given, dtype=torch.float32, device="cuda")
    mp, kp = native.round128(x.shape[0]), native.round128(x.shape[1])
    packed, scales, pts = native.quantize(xd, signs, mp, kp, 2 if sr else 0, rht, seed, given_scale=scale)
    assert np.float32(pts.item()) == np.float32(want[2])
    _cmp(packed, scales, want)


def test_weight_pair_matches_reference_cuda_kernel(native, golden_cuda_quant):
    g = golden_cuda_quant
    w = torch.from_numpy(g["pair_w"]).cuda()
    pts = torch.from_numpy(g["pair_pts"]).cuda()
    mp, kp = native.round128(w.shape[0]), native.round128(w.shape[1])
    d, s, p, dt, st = native.quantize(w, signs_dev(), mp, kp, 0, False, 0, given_scale=pts.reshape(()), pair=True)
    _cmp(d, s, (g["pair_data"], g["pair_scale"]))
    _cmp(dt, st, (g["pair_data_t"], g["pair_scale_t"]))
    assert np.float32(native.amax(w)[1].item()) == g["pair_pts"][0]


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("rht", [False, True])
def test_one_launch_operator_equals_amax_then_quantise(native, mode, rht):
    """BF16 tensors that fit shared memory take amax, scale and packing in one cooperative launch; the result is the
    two-launch result (amax kernel, then the quantiser with that scale) byte for byte, on repeated calls (the barrier
    words return to zero), under graph replay, and next to a tensor just above the size limit that takes two launches."""
    flag, _ = MODES[mode]
    signs = signs_dev()
    for shape in ((4096, 4096), (1024, 640), (300, 1000), (4224, 4096)):
        x = outlier_tensor(shape, seed=shape[0] + shape[1]).cuda()
        mp, kp = native.round128(shape[0]), native.round128(shape[1])
        four = native.amax(x).clone()
        scale = four[2 if rht else 1].clone()
        want = native.quantize(x, signs, mp, kp, flag, rht, 11, given_scale=scale)
        for _ in range(3):
            got = native.quantize(x, signs, mp, kp, flag, rht, 11)
            assert torch.equal(got[2], scale)
            assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    x = outlier_tensor((2048, 2048), seed=3).cuda()
    want = native.quantize(x, signs, 2048, 2048, flag, rht, 5)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        native.quantize(x, signs, 2048, 2048, flag, rht, 5)      # scratch of this stream exists before the capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        got = native.quantize(x, signs, 2048, 2048, flag, rht, 5)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    native.check_status()
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
