"""tcgen05 block-scaled GEMM through the C ABI against the CPU oracle.

Bit patterns of a GEMM are not pinned by the reference (its GEMM is a cuBLASLt call whose accumulation order
is unspecified); the contract is: relative Frobenius error <= 1e-2 against a BF16 matmul of the dequantised
operands.  The kernel is held to a much tighter bound against the exact (float64) block-scaled product."""
import numpy as np
import pytest
import torch

import oracle as O
from _util import signs_dev

pytestmark = pytest.mark.gpu

SHAPES = [(128, 128, 128), (128, 256, 256), (256, 128, 384), (128, 384, 512), (384, 512, 1024), (256, 256, 2048),
          (1024, 1024, 640)]


def _operands(native, m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g).bfloat16().cuda()
    w = (torch.randn((n, k), generator=g) * 0.05).bfloat16().cuda()
    sg = signs_dev()
    a = native.quantize(x, sg, native.round128(m), native.round128(k), 0, False, 0)
    b = native.quantize(w, sg, native.round128(n), native.round128(k), 0, False, 0)
    return a, b


def _exact(a, b):
    da = torch.from_numpy(O.decode_unscaled(a[0].cpu().numpy(), a[1].cpu().numpy())).double()
    db = torch.from_numpy(O.decode_unscaled(b[0].cpu().numpy(), b[1].cpu().numpy())).double()
    return da @ db.t()


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_fp32_raw_matches_exact_product(native, m, n, k):
    a, b = _operands(native, m, n, k, seed=m + n + k)
    out = native.gemm(a[0], a[1], None, b[0], b[1], None, rows=a[0].shape[0], cols=b[0].shape[0], out_dtype=torch.float32, raw_bf16=False)
    native.check_status()
    want = _exact(a, b)
    got = out.double().cpu()
    rel = (got - want).norm() / want.norm()
    assert rel < 2e-6, rel
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-3 * want.abs().max().item())


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (200, 300, 500), (65, 67, 131), (384, 512, 1024)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_epilogue_matches_reference_rounding_chain(native, m, n, k, out_dtype, with_bias):
    a, b = _operands(native, m, n, k, seed=7 * m + n)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16 if out_dtype == torch.bfloat16 else torch.float32)
    out = native.gemm(a[0], a[1], a[2], b[0], b[1], b[2], rows=m, cols=n, out_dtype=out_dtype, bias=bias.cuda() if with_bias else None)
    native.check_status()
    assert out.shape == (m, n)
    pa = (a[0].cpu().numpy(), a[1].cpu().numpy(), float(a[2].item()))
    pb = (b[0].cpu().numpy(), b[1].cpu().numpy(), float(b[2].item()))
    want = O.matmul_packed(pa, pb, m, n, raw_bf16=True, out_bf16=out_dtype == torch.bfloat16, bias=bias.float().numpy() if with_bias else None)
    got = out.float().cpu().numpy()
    # the accumulator is rounded to BF16 first: summation order can move a value across a rounding boundary,
    # so allow one BF16 step on a small fraction of the elements and require the rest to be identical
    step = np.abs(want) * 2.0 ** -7 + 1e-12
    assert (np.abs(got - want) <= 1.01 * step).all()
    assert (got == want).mean() > 0.98
    # the contract of the benchmark configs: <= 1e-2 relative Frobenius vs a BF16 matmul of the dequantised operands
    da = torch.from_numpy(O.dequantize(pa[0], pa[1], pa[2], m, k)).bfloat16()
    db = torch.from_numpy(O.dequantize(pb[0], pb[1], pb[2], n, k)).bfloat16()
    ref = (da.float() @ db.float().t()).numpy() + (bias.float().numpy() if with_bias else 0.0)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-2


def test_gemm_roles_of_a_linear_layer(native):
    """fprop, dgrad and wgrad of one layer use the same kernel on different packings."""
    g = torch.Generator().manual_seed(1234)
    tokens, d_in, d_out = 512, 384, 256
    x = torch.randn((tokens, d_in), generator=g).bfloat16().cuda()
    w = (torch.randn((d_out, d_in), generator=g) * 0.02).cuda()
    gy = (torch.randn((tokens, d_out), generator=g) * 1e-3).bfloat16().cuda()
    sg = signs_dev()
    xq = native.quantize(x, sg, 512, 384, 0, False, 0)
    wq = native.quantize(w, sg, 256, 384, 0, False, 0, pair=True)
    y = native.gemm(xq[0], xq[1], xq[2], wq[0], wq[1], wq[2], rows=tokens, cols=d_out)
    gq = native.quantize(gy, sg, 512, 256, 2, False, 1234)
    dx = native.gemm(gq[0], gq[1], gq[2], wq[3], wq[4], wq[2], rows=tokens, cols=d_in)
    gt = native.quantize(gy.t(), sg, 256, 512, 2, True, 1235)
    xt = native.quantize(x.t(), sg, 384, 512, 0, True, 0)
    dw = native.gemm(gt[0], gt[1], gt[2], xt[0], xt[1], xt[2], rows=d_out, cols=d_in, out_dtype=torch.float32, raw_bf16=False)
    native.check_status()
    xf, wf, gf = x.float(), w.bfloat16().float(), gy.float()
    for got, want in ((y.float(), xf @ wf.t()), (dx.float(), gf @ wf), (dw, gf.t() @ xf)):
        rel = (got - want).norm() / want.norm()
        assert rel < 0.2, rel  # FP4 quantisation noise of random Gaussians; the kernel itself is checked above


def test_gemm_argument_errors(native):
    z = torch.zeros((128, 64), dtype=torch.uint8, device="cuda")
    s = torch.zeros((32, 32), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        native.gemm(z[:100], s, None, z, s, None, rows=100, cols=128)
    with pytest.raises(ValueError):
        native.gemm(z, s, None, z, s, None, rows=129, cols=128)


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("m,n,k,rows,cols", [(256, 512, 128, 256, 512), (512, 256, 1024, 500, 250), (256, 256, 384, 255, 129),
                                             (4096, 4096, 256, 4096, 4096), (2048, 4096, 640, 2048, 4090)])
@pytest.mark.parametrize("mode", ["bf16", "bf16_bias", "fp32_bias", "fp32_alpha_bf16"])
def test_gemm_paired_and_single_forms_agree_with_the_oracle(native, pair, m, n, k, rows, cols, mode):
    """Shapes whose M and N are multiples of 256 run on clusters of two CTAs unless told otherwise; both forms must give
    the oracle's bits in every epilogue (fast BF16, bias chain, FP32 output, FP32 alpha), with cropped and unaligned
    outputs, one-k-tile contractions and several tiles per CTA (the two overlapping accumulator stages alternate)."""
    a, b = _operands(native, m, n, k, seed=3 * m + n + k)
    out_dtype = torch.float32 if mode == "fp32_bias" else torch.bfloat16
    raw_bf16 = mode != "fp32_alpha_bf16"
    bias = None
    if mode.endswith("bias"):
        bias = (torch.randn(cols, generator=torch.Generator().manual_seed(5)) * 0.5).to(out_dtype)
    out = native.gemm(a[0], a[1], a[2], b[0], b[1], b[2], rows=rows, cols=cols, out_dtype=out_dtype, raw_bf16=raw_bf16,
                      bias=None if bias is None else bias.cuda(), pair=pair)
    native.check_status()
    assert out.shape == (rows, cols)
    pa = (a[0].cpu().numpy(), a[1].cpu().numpy(), float(a[2].item()))
    pb = (b[0].cpu().numpy(), b[1].cpu().numpy(), float(b[2].item()))
    want = O.matmul_packed(pa, pb, rows, cols, raw_bf16=raw_bf16, out_bf16=out_dtype == torch.bfloat16,
                           bias=None if bias is None else bias.float().numpy())
    got = out.float().cpu().numpy()
    step = np.abs(want) * 2.0 ** -7 + 1e-12
    assert (np.abs(got - want) <= 1.01 * step).all()
    assert (got == want).mean() > 0.98


# ---- the benchmark configurations' own shapes -------------------------------------------------------------------------
# (M, N, K) of out[M, N] = A[M, K] B[N, K]^T.  Linear-layer config: X[8192, 4096], W[4096, 4096]: fprop / dgrad and the
# weight gradient, whose contraction runs over the 8192 tokens.  Decoder config (d 3072, FFN 8192, 8192 tokens): q/k/v/o
# and down fprop, gate/up fprop, their dgrads and the three wgrad shapes.
BASELINE_SHAPES = [(8192, 4096, 4096), (4096, 4096, 8192), (8192, 3072, 3072), (8192, 8192, 3072), (8192, 3072, 8192),
                   (3072, 8192, 8192)]
_BIG = {}


def _big_case(native, m, n, k):
    """Operands quantised on the GPU once per shape, with their oracle decodings (unscaled, and dequantised BF16)."""
    key = (m, n, k)
    if key not in _BIG:
        _BIG.clear()   # one shape's worth of host memory at a time
        a, b = _operands(native, m, n, k, seed=m + 3 * n + 7 * k)
        host = [(t[0].cpu().numpy(), t[1].cpu().numpy(), float(t[2].item())) for t in (a, b)]
        ua, ub = (O.decode_unscaled(h[0], h[1]) for h in host)
        da = torch.from_numpy(O.dequantize(host[0][0], host[0][1], host[0][2], m, k)).bfloat16().cuda()
        db = torch.from_numpy(O.dequantize(host[1][0], host[1][1], host[1][2], n, k)).bfloat16().cuda()
        ref = (da @ db.t()).float()     # the BF16 matmul of the dequantised operands the accuracy criterion names
        _BIG[key] = (a, b, host, ua, ub, ref)
    return _BIG[key]


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("scaled", [True, False])
@pytest.mark.parametrize("m,n,k", BASELINE_SHAPES)     # outermost: the four variants of a shape share its operands
def test_gemm_at_benchmark_shapes(native, m, n, k, pair, scaled):
    """Full-size GEMMs of the benchmark configurations (up to 32 k-tiles, several tiles per CTA with the accumulator stages
    alternating): relative Frobenius error <= 1e-2 against a BF16 matmul of the oracle-dequantised operands over the
    whole output, and the oracle's bits on a strided sample of rows and columns.  scaled=False is the raw BF16
    accumulator image the optimizer decodes (no tensor scales)."""
    a, b, host, ua, ub, ref = _big_case(native, m, n, k)
    pts_a, pts_b = (a[2], b[2]) if scaled else (None, None)
    out = native.gemm(a[0], a[1], pts_a, b[0], b[1], pts_b, rows=m, cols=n, out_dtype=torch.bfloat16, raw_bf16=True, pair=pair)
    native.check_status()
    got = out.float()
    if scaled:
        rel = ((got - ref).norm() / ref.norm()).item()
        assert rel < 1e-2, rel
    else:
        alpha = host[0][2] * host[1][2]
        rel = ((got * alpha - ref).norm() / ref.norm()).item()
        assert rel < 1e-2, rel
    ri = np.unique(np.concatenate([np.arange(0, m, 149), [127, 128, 255, 256, m - 129, m - 1]]))
    ci = np.unique(np.concatenate([np.arange(0, n, 131), [127, 128, 255, 256, n - 129, n - 1]]))
    raw = (torch.from_numpy(ua[ri]).double() @ torch.from_numpy(ub[ci]).double().t()).float().numpy()
    sa, sb = (host[0][2], host[1][2]) if scaled else (1.0, 1.0)
    want = O.rescale(raw, sa, sb, len(ri), len(ci), raw_bf16=True, out_bf16=True)
    sample = got[torch.from_numpy(ri).cuda()][:, torch.from_numpy(ci).cuda()].cpu().numpy()
    step = np.abs(want) * 2.0 ** -7 + 1e-12
    assert (np.abs(sample - want) <= 1.01 * step).all()
    assert (sample == want).mean() > 0.98
