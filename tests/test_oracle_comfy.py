"""CPU checks of the packed-checkpoint (Comfy order) oracle: scalar functions against vectors produced by the
reference's own device functions, and the relations the reference's tests state for the kernels built from them."""
import numpy as np
import pytest

import oracle as O
from conftest import GOLDEN


@pytest.fixture(scope="module")
def scalars():
    return np.load(GOLDEN / "comfy_scalar_reference.npz")


def test_scalar_functions_match_reference_vectors(scalars):
    L, d = O.lib(), scalars
    got = np.array([L.orc_comfy_bf(int(v)) for v in d["bf_in"]], dtype=np.float32).view(np.uint32)
    assert np.array_equal(got, d["bf_out"])
    rb_in = d["rb_in"].view(np.float32)
    assert np.array_equal(np.array([L.orc_comfy_rb(float(v)) for v in rb_in], dtype=np.uint16), d["rb_out"])
    assert np.array_equal(np.array([L.orc_comfy_f8(int(v)) for v in d["f8_in"]], dtype=np.float32)[:127], d["f8_out"][:127])
    assert np.array_equal(np.array([L.orc_comfy_f8(int(v)) for v in d["f8_in"]], dtype=np.float32).view(np.uint32),
                          d["f8_out"].view(np.uint32))
    assert np.array_equal(np.array([L.orc_comfy_rf8(float(v)) for v in d["rf8_in"]], dtype=np.uint8), d["rf8_out"])
    assert np.array_equal(np.array([L.orc_comfy_f4(int(v)) for v in d["f4_in"]], dtype=np.float32).view(np.uint32),
                          d["f4_out"].view(np.uint32))
    assert np.array_equal(np.array([L.orc_comfy_mix(int(v)) for v in d["mix_in"]], dtype=np.uint32), d["mix_out"])
    for sr in (0, 1):
        got = np.array([L.orc_comfy_rf4(float(v), int(r), sr) for v, r in zip(d["rf4_v"], d["rf4_rng"])], dtype=np.uint8)
        assert np.array_equal(got, d[f"rf4_out_sr{sr}"]), sr
    got = np.array([L.orc_comfy_swizzle(int(r), int(b), int(k)) for r, b, k in zip(d["sw_r"], d["sw_b"], d["sw_k"])])
    assert np.array_equal(got, d["sw_out"])


def test_hardware_rne_model_equals_reference_software_rne(scalars):
    """The reference's rf4 with sr = 0 is its software statement of round-to-nearest-even; the quantiser uses the
    hardware conversion instead (_packed_cuda.py:48-52).  Both must choose the same code for every finite input."""
    L = O.lib()
    v = scalars["rf4_v"]
    hw = np.array([L.orc_f32_to_e2m1_rne(float(x)) for x in v], dtype=np.uint8)
    assert np.array_equal(hw, scalars["rf4_out_sr0"])


def test_swizzle_is_the_shared_scale_layout():
    """For widths that are multiples of 64 the packed backend and the training quantiser address scale bytes alike,
    which is what lets one GEMM kernel serve both."""
    L = O.lib()
    for k in (64, 128, 320, 4096):
        for r in (0, 1, 31, 32, 127, 128, 300):
            for b in range(0, k // 16, 3):
                assert L.orc_comfy_swizzle(r, b, k) == L.orc_scale_offset(r, b * 16, k)


def test_finish_scale_is_the_correctly_rounded_quotient():
    # tests/test_packed_lora.py:40-44 of the reference: float32(amax / 2688) computed in float64, floor 1e-30
    L = O.lib()
    for amax in (0.0, 1.0872942, 1.0872943, 1.0, 0.001, 10000.0):
        want = max(np.float32(np.float64(np.float32(amax)) / 2688.0), np.float32(1e-30))
        assert np.float32(L.orc_comfy_finish_scale(amax)) == want


def _weights(n, k, seed, outliers=True):
    rng = np.random.default_rng(seed)
    w = rng.standard_normal((n, k)).astype(np.float32) * 0.02
    if outliers:
        w.flat[rng.integers(0, w.size, max(1, w.size // 1000))] *= 30
    return O.to_bf16_bits(w)


def test_quantise_dequantise_round_trip_error():
    x = _weights(48, 256, 3)
    q, s, g = O.comfy_quantize(x)
    back = O.from_bf16_bits(O.comfy_dequantize(q, s, g))[:48]
    ref = O.from_bf16_bits(x)
    rel = np.linalg.norm(back - ref) / np.linalg.norm(ref)
    assert rel < 0.12
    assert q.shape == (48, 128) and s.size == 128 * 16
    # zero rows stay zero, including the rows padded to a multiple of 16
    x[5] = 0
    q2, s2, _ = O.comfy_quantize(x[:40])
    assert q2.shape[0] == 48 and not q2[40:].any() and not q2[5].any()


def test_rotation_is_orthonormal_and_an_involution_up_to_signs():
    rng = np.random.default_rng(0)
    x = O.to_bf16_bits(rng.standard_normal((4, 256)).astype(np.float32))
    signs = O.comfy_signs(5)
    y = np.zeros((4, 256), dtype=np.float32)
    amax = O.lib().orc_comfy_rotate(x.ctypes.data, signs.ctypes.data, y.ctypes.data, 4, 256)
    xf = O.from_bf16_bits(x)
    assert abs(np.linalg.norm(y) - np.linalg.norm(xf)) < 1e-4 * np.linalg.norm(xf)
    assert amax == np.abs(y).max()
    # against the dense Sylvester matrix
    h = np.array([[1.0]])
    for _ in range(7):
        h = np.block([[h, h], [h, -h]])
    dense = (xf.reshape(-1, 128) * signs) @ h / np.sqrt(128)
    assert np.allclose(np.abs(dense), np.abs(y.reshape(-1, 128)), atol=2e-5)
    assert np.allclose(dense, y.reshape(-1, 128), atol=2e-5)


@pytest.mark.parametrize("n,k", [(128, 128), (256, 384)])
def test_transpose_requant_equals_quantise_of_dequantised_transpose(n, k):
    """tests/test_packed_lora.py:46-52 of the reference: the packed -> packed kernel gives the same bytes as
    dequantise, transpose, rotate + quantise with the separately computed backward scale."""
    w = _weights(n, k, 11)
    q, s, g = O.comfy_quantize(w)
    signs = O.comfy_signs(9)
    bscale = O.comfy_backward_scale(q, s, g, signs)
    qt, st = O.comfy_transpose_requant(q, s, g, signs, bscale)
    dense_t = np.ascontiguousarray(O.comfy_dequantize(q, s, g).T)
    q2, s2, g2 = O.comfy_quantize(dense_t, signs)
    assert g2 == bscale
    assert np.array_equal(q2, qt) and np.array_equal(s2, st)


def test_stochastic_rounding_is_unbiased_and_seeded():
    rng = np.random.default_rng(2)
    x = O.to_bf16_bits(rng.standard_normal((64, 128)).astype(np.float32))
    ref = O.from_bf16_bits(x)
    acc = np.zeros_like(ref)
    first = None
    for seed in range(64):
        q, s, g = O.comfy_quantize(x, sr=True, seed=seed)
        if first is None:
            first = q.copy()
            assert np.array_equal(O.comfy_quantize(x, sr=True, seed=seed)[0], first)
        acc += O.from_bf16_bits(O.comfy_dequantize(q, s, g))
    assert not np.array_equal(O.comfy_quantize(x, sr=True, seed=1)[0], first)
    one = O.from_bf16_bits(O.comfy_dequantize(*O.comfy_quantize(x)))
    err_mean = np.linalg.norm(acc / 64 - ref) / np.linalg.norm(ref)
    err_one = np.linalg.norm(one - ref) / np.linalg.norm(ref)
    assert err_mean < 0.35 * err_one


def test_rope_backward_is_the_transpose():
    rng = np.random.default_rng(4)
    rows, heads, dim, pairs = 5, 2, 16, 6
    x = O.to_bf16_bits(rng.standard_normal((1, rows, heads, dim)).astype(np.float32))
    g = O.to_bf16_bits(rng.standard_normal((1, rows, heads, dim)).astype(np.float32))
    rot = O.to_bf16_bits(rng.standard_normal((rows, pairs, 2, 2)).astype(np.float32))
    y = O.from_bf16_bits(O.comfy_rope(x, rot, pairs))
    gx = O.from_bf16_bits(O.comfy_rope(g, rot, pairs, backward=True))
    xf, gf = O.from_bf16_bits(x), O.from_bf16_bits(g)
    assert abs((y * gf).sum() - (xf * gx).sum()) < 0.05 * np.abs(y * gf).sum()
    assert np.array_equal(y[..., 2 * pairs:], xf[..., 2 * pairs:])
