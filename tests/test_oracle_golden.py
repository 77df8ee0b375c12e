"""The CPU oracle against golden vectors produced by the reference's own Triton kernels
(tests/golden/make_golden.py) and against published / library known answers."""
import numpy as np
import pytest
import torch

import oracle as O

DUAL = ["a", "b", "c", "d", "e", "f"]


def _src(blob, key, is_bf16):
    x = blob[key]
    return x  # uint16 bit patterns (bf16) or float32


@pytest.mark.parametrize("tag", DUAL)
def test_dual_matches_reference(golden_quant, tag):
    g = golden_quant
    sr, seed, is_bf16 = (int(v) for v in g[f"dual_{tag}_meta"])
    x = g[f"dual_{tag}_x"]
    row, col = O.dual(x, sr_mode=O.SR_HASH if sr else O.RNE, signs=g["signs"], seed=seed)
    for name, got in (("row", row), ("col", col)):
        assert np.float32(got[2]) == g[f"dual_{tag}_{name}_pts"][0]
        assert np.array_equal(got[0], g[f"dual_{tag}_{name}_data"]), f"{name} payload"
        assert np.array_equal(got[1], g[f"dual_{tag}_{name}_scale"]), f"{name} scales"


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_weight_pair_and_single_match_reference(golden_quant, tag):
    g = golden_quant
    kind = {0: None, 1: None, 2: "f16"}[int(g[f"pair_{tag}_kind"][0])]
    w, pts = g[f"pair_{tag}_w"], float(g[f"pair_{tag}_pts"][0])
    row, col = O.weight_pair(w, pts_value=pts, kind=kind)
    assert np.array_equal(row[0], g[f"pair_{tag}_data"]) and np.array_equal(row[1], g[f"pair_{tag}_scale"])
    assert np.array_equal(col[0], g[f"pair_{tag}_data_t"]) and np.array_equal(col[1], g[f"pair_{tag}_scale_t"])
    assert np.array_equal(row[0], g[f"single_{tag}_0_data"]) and np.array_equal(row[1], g[f"single_{tag}_0_scale"])
    assert np.array_equal(col[0], g[f"single_{tag}_1_data"]) and np.array_equal(col[1], g[f"single_{tag}_1_scale"])
    # the tensor scale the optimizer caches: max(amax,1e-12) * (1/2688)  (optimizer_v5.py:64)
    assert np.float32(O.pts(O.amax(w, kind=kind), 1.0)) == np.float32(pts)


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_rescale_matches_reference(golden_quant, tag):
    g = golden_quant
    raw_bf16, out_bf16, with_bias = (bool(v) for v in g[f"rescale_{tag}_meta"])
    raw = g[f"rescale_{tag}_raw"]
    raw = O.from_bf16_bits(raw) if raw_bf16 else raw
    sa, sb = (float(v) for v in g[f"rescale_{tag}_scales"])
    bias = g[f"rescale_{tag}_bias"] if with_bias else None
    out = O.rescale(raw, sa, sb, 100, 200, raw_bf16=raw_bf16, out_bf16=out_bf16, bias=bias)
    assert np.array_equal(out.view(np.uint32), g[f"rescale_{tag}_out"].view(np.uint32))


def _cuda_quant_names():
    from conftest import GOLDEN
    return [str(n) for n in np.load(GOLDEN / "cuda_quant_reference.npz")["names"]]


@pytest.mark.parametrize("name", _cuda_quant_names())
def test_quantize_matches_reference_cuda_kernels(golden_cuda_quant, name):
    """quantize_cuda (csrc/kernels.cu:237-298) with quant_rows / quant_transpose / emit_group run on the host: row and
    transposed orientation, strided views, SR x RHT, tensor scale (factor * max(amax, 1e-12)) * (1 / 2688)."""
    from conftest import cuda_quant_case
    x, sr, rht, seed, given, want = cuda_quant_case(golden_cuda_quant, name)
    xn = x.view(torch.int16).numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.numpy()
    got = O.quantize(xn, sr_mode=O.SR_HASH if sr else O.RNE, rht=rht, signs=golden_cuda_quant["signs"], seed=seed, pts_value=given)
    assert np.float32(got[2]) == np.float32(want[2])
    assert np.array_equal(got[1], want[1]), "scales"
    assert np.array_equal(got[0], want[0]), "payload"


def test_weight_pair_matches_reference_cuda_kernel(golden_cuda_quant):
    """quant_weight_pair (csrc/kernels.cu:165-185)."""
    g = golden_cuda_quant
    row, col = O.weight_pair(g["pair_w"], pts_value=float(g["pair_pts"][0]))
    assert np.array_equal(row[0], g["pair_data"]) and np.array_equal(row[1], g["pair_scale"])
    assert np.array_equal(col[0], g["pair_data_t"]) and np.array_equal(col[1], g["pair_scale_t"])


def test_hardware_stochastic_conversion_model():
    """The oracle's model of cvt.rs.satfinite.e2m1x4.f32 against the instruction's outputs recorded on a B200
    (tests/golden/cvt_rs_probe.cu): single operands against every byte of the random word, and random quadruples."""
    from conftest import GOLDEN
    g = np.load(GOLDEN / "cvt_rs_e2m1x4.npz")
    L = O.lib()
    got = np.array([L.orc_cvt_rs_e2m1x4(float(a), float(b), float(c), float(d), int(r))
                    for a, b, c, d, r in zip(g["a"], g["b"], g["c"], g["d"], g["rbits"])], dtype=np.uint16)
    assert np.array_equal(got, g["out"])


def test_philox_known_answers():
    # Random123 known-answer vectors for philox4x32-10
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
            [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        assert [int(v) for v in O.philox(ctr, key)] == want


def test_scalar_formats_match_torch_cpu():
    L = O.lib()
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.rand(4000, generator=g) * 500, torch.rand(4000, generator=g) * 0.05, torch.tensor([0.0, 448.0, 0.015625, 2.0 ** -9])])
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([L.orc_f32_to_e4m3(float(v)) for v in x.numpy()], dtype=np.uint8)
    ok = (got == want) | (x.numpy() > 448)  # above 448 the oracle saturates like cvt.rn.satfinite; torch gives NaN
    assert ok.all()
    assert all(L.orc_f32_to_e4m3(v) == 0x7e for v in (449.0, 464.0, 1e9))
    y = torch.randn(4000, generator=g) * torch.tensor(10.0) ** torch.randint(-9, 5, (4000,), generator=g).float()
    want16 = y.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(np.array([L.orc_f32_to_f16(float(v)) for v in y.numpy()], dtype=np.uint16), want16)
    assert np.array_equal(O.to_bf16_bits(y.numpy()), y.bfloat16().view(torch.int16).numpy().view(np.uint16))


def test_e2m1_rne_ties_to_even_code():
    L = O.lib()
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6, 7.0: 7, 0.26: 1, 5.01: 7}
    for v, code in ties.items():
        assert L.orc_f32_to_e2m1_rne(v) == code
        assert L.orc_f32_to_e2m1_rne(-v) == code | 8


def test_zero_stays_zero_and_scale_floor():
    # verify_fast_v2.py:70-73 — an all-zero tensor encodes to zero payload with the minimum block scale
    x = np.zeros((17, 35), dtype=np.float32)
    for sr in (O.RNE, O.SR_HASH, O.SR_PHILOX):
        for rht in (False, True):
            p, s, t = O.quantize(x, sr_mode=sr, rht=rht, seed=3)
            assert not p.any() and (s == 0x08).all()
            assert not O.dequantize(p, s, t, 17, 35).any()


def test_finish_scale_variants():
    # tests/test_packed_lora.py:40-44 — the packed backend's scale is a correctly rounded division
    for a in (0.0, 1.0872942, 1.0872943, 1.0, 0.001, 10000.0):
        want = max(np.float32(np.float64(np.float32(a)) / 2688.0), np.float32(1e-30))
        assert np.float32(O.pts(a, 1.0, 2)) == want


def test_sr_is_unbiased_and_seeded():
    # verify_fast_v2.py:79-95 — different seeds differ; averaging SR samples beats one sample
    g = np.random.default_rng(0)
    x = g.standard_normal((128, 128)).astype(np.float32)
    ref = O.from_bf16_bits(O.to_bf16_bits(x))
    for mode in (O.SR_HASH, O.SR_PHILOX):
        outs = []
        for seed in range(32):
            p, s, t = O.quantize(x, sr_mode=mode, seed=seed)
            outs.append(O.dequantize(p, s, t, 128, 128))
        assert not np.array_equal(outs[0], outs[1])
        single = np.abs(outs[0] - ref).mean()
        mean = np.abs(np.mean(outs, axis=0) - ref).mean()
        assert mean < 0.55 * single
        again = O.quantize(x, sr_mode=mode, seed=0)
        assert np.array_equal(O.dequantize(*again, 128, 128), outs[0])


def test_transposed_view_equals_explicit_transpose():
    g = np.random.default_rng(1)
    x = g.standard_normal((193, 129)).astype(np.float32)
    a = O.quantize(x, transpose=True, rht=True, sr_mode=O.SR_HASH, seed=9)
    b = O.quantize(np.ascontiguousarray(x.T), rht=True, sr_mode=O.SR_HASH, seed=9)
    assert all(np.array_equal(u, v) for u, v in zip(a[:2], b[:2])) and a[2] == b[2]
    strided = g.standard_normal((260, 600)).astype(np.float32)[::2, ::2]
    c = O.quantize(strided)
    d = O.quantize(np.ascontiguousarray(strided))
    assert all(np.array_equal(u, v) for u, v in zip(c[:2], d[:2]))


def test_rht_dequantised_error_is_small():
    # verify_fast_v2.py:35-76 thresholds: dequantised relative error <= 0.005 of the rotated input
    g = np.random.default_rng(2)
    x = g.standard_normal((128, 256)).astype(np.float32)
    signs = O.default_signs()
    p, s, t = O.quantize(x, rht=True, signs=signs)
    xb = O.from_bf16_bits(O.to_bf16_bits(x)).reshape(128, 16, 16) * signs
    import scipy.linalg
    h = scipy.linalg.hadamard(16).astype(np.float32)
    want = (xb @ h * 0.25).reshape(128, 256)
    got = O.dequantize(p, s, t, 128, 256)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel < 0.12  # FP4 quantisation noise of a Gaussian; sanity bound on the rotation itself
    assert abs(np.linalg.norm(want) / np.linalg.norm(xb.reshape(128, 256)) - 1) < 1e-5
