"""Launchers of the packed-checkpoint kernels: the functions of the reference's src/precision_lora/_packed_cuda.py
(dequant :221-225, quantize :228-243, matmul :245-250, rope :251-264, transpose_rht_quant :266-273, backward_scale
:276-287) with the same names, arguments and results, over the prebuilt sm_100a library instead of NVRTC-compiled
SM120 code and over this package's tcgen05 GEMM instead of the cuBLASLt call.

A quantised tensor is the tuple (payload uint8 [rows, cols / 2] with the even element in the high nibble,
E4M3 block scales in the 128 x 4 swizzle, FP32 tensor scale)."""
import torch

from nvfp4_training import _native as nat


def init():
    """Device gate (the reference requires SM120 here, this build requires compute capability 10.x)."""
    from nvfp4_training._runtime import load_runtime
    load_runtime()


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def dequant(q, s, g):
    init()
    n, k = q.shape[0], q.shape[1] * 2
    out = torch.empty((n, k), device=q.device, dtype=torch.bfloat16)
    with torch.cuda.device(q.device):
        nat.check(nat.lib().nvfp4_comfy_dequantize(q.data_ptr(), s.data_ptr(), g.data_ptr(), out.data_ptr(), n, k, _stream(q)))
    return out


def quantize(x, signs=None, seed=0, sr=False):
    """BF16 [n, k], k % 128 == 0 -> (q [ceil16(n), k / 2], scales [ceil128(n), k / 16] E4M3, tensor scale).
    `signs` (128 floats, +-1) selects the H128 rotation; `seed` is an int, or an int32 device tensor read by the
    kernel so that graph replays see its current value."""
    init()
    n, k = x.shape
    if not (x.is_cuda and x.is_contiguous() and k % 128 == 0 and x.dtype == torch.bfloat16):
        raise AssertionError("quantize expects a contiguous CUDA BF16 matrix whose width is a multiple of 128")
    rows16, rows128 = (n + 15) // 16 * 16, (n + 127) // 128 * 128
    # the payload owns whole 128-row tiles (what the GEMM's tensor map walks); the result is the ceil16 view
    q = torch.empty((rows128, k // 2), dtype=torch.uint8, device=x.device)[:rows16]
    s = torch.empty((rows128, k // 16), dtype=torch.float8_e4m3fn, device=x.device)
    g = torch.empty((), dtype=torch.float32, device=x.device)
    amax = torch.empty((), dtype=torch.float32, device=x.device)
    on_device = torch.is_tensor(seed)
    with torch.cuda.device(x.device):
        nat.check(nat.lib().nvfp4_comfy_quantize(x.data_ptr(), n, k, nat.ptr(signs), int(bool(sr)),
                                                 0 if on_device else int(seed) & 0xFFFFFFFF,
                                                 seed.data_ptr() if on_device else None, q.data_ptr(), s.data_ptr(),
                                                 g.data_ptr(), amax.data_ptr(), _stream(x)))
    return q, s, g


def matmul(a, b, dtype=torch.bfloat16, rows=None, cols=None):
    """a @ b.T for two quantised tensors: FP32 accumulation, one multiplication by g_a * g_b, one rounding to `dtype`.
    The nibble order inside a byte does not matter to the product as long as both operands share it.  `rows` / `cols`
    crop the result inside the kernel's epilogue (default: the payload row counts, as the reference returns)."""
    init()
    (qa, sa, ga), (qb, sb, gb) = a, b
    rows = qa.shape[0] if rows is None else rows
    cols = qb.shape[0] if cols is None else cols
    return nat.gemm(_whole_tiles(qa), sa, ga, _whole_tiles(qb), sb, gb, rows=rows, cols=cols, out_dtype=dtype, raw_bf16=False)


def _whole_tiles(q):
    """The payload with its row count rounded up to 128: the view over the allocation quantize() made when there is
    one, else a zero-padded copy.  Rows past the logical end carry zero block scales, so their content is irrelevant."""
    rows, width = q.shape
    padded = (rows + 127) // 128 * 128
    if padded == rows:
        return q
    if q.is_contiguous() and q.storage_offset() == 0 and q.untyped_storage().nbytes() >= padded * width:
        return torch.empty(0, dtype=torch.uint8, device=q.device).set_(q.untyped_storage(), 0, (padded, width), (width, 1))
    return torch.nn.functional.pad(q, (0, 0, 0, padded - rows))


def _rope(x, rotation, backward=False):
    init()
    assert x.ndim == 4 and x.shape[0] == 1 and x.dtype == torch.bfloat16 and rotation.dtype == torch.bfloat16
    x, rotation = x.contiguous(), rotation.contiguous()
    out = torch.empty_like(x)
    _, rows, heads, dim = x.shape
    pairs = rotation.shape[-3]
    with torch.cuda.device(x.device):
        nat.check(nat.lib().nvfp4_comfy_rope(x.data_ptr(), rotation.data_ptr(), out.data_ptr(), rows, heads, dim, pairs,
                                             int(backward), _stream(x)))
    return out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rotation):
        assert not rotation.requires_grad
        ctx.save_for_backward(rotation)
        return _rope(x, rotation)

    @staticmethod
    def backward(ctx, g):
        return _rope(g, ctx.saved_tensors[0], True), None


def rope(x, rotation):
    return _RopeFn.apply(x, rotation)


def transpose_rht_quant(source, signs, backward_scale):
    """Packed [n, k] -> (packed rotated [k, n / 2], scales [k, n / 16], backward_scale) without a dense copy."""
    init()
    q, s, g = source
    n, k = q.shape[0], q.shape[1] * 2
    assert n % 128 == 0 and k % 128 == 0
    qt = torch.empty((k, n // 2), device=q.device, dtype=torch.uint8)
    st = torch.empty((k, n // 16), device=q.device, dtype=torch.float8_e4m3fn)
    with torch.cuda.device(q.device):
        nat.check(nat.lib().nvfp4_comfy_transpose_requant(q.data_ptr(), s.data_ptr(), g.data_ptr(), signs.data_ptr(),
                                                          backward_scale.data_ptr(), qt.data_ptr(), st.data_ptr(), n, k,
                                                          _stream(q)))
    return qt, st, backward_scale


def backward_scale(source, signs):
    """Tensor scale of the rotated transpose, max(amax / 2688, 1e-30), with the division done on the device so it
    is the same operation the quantiser uses."""
    init()
    q, s, g = source
    n, k = q.shape[0], q.shape[1] * 2
    assert n % 128 == 0 and k % 128 == 0
    amax = torch.empty((), device=q.device, dtype=torch.float32)
    scale = torch.empty((), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        nat.check(nat.lib().nvfp4_comfy_backward_scale(q.data_ptr(), s.data_ptr(), g.data_ptr(), signs.data_ptr(), n, k,
                                                       amax.data_ptr(), scale.data_ptr(), _stream(q)))
    return scale


def finish_scale(amax):
    init()
    scale = torch.empty((), device=amax.device, dtype=torch.float32)
    with torch.cuda.device(amax.device):
        nat.check(nat.lib().nvfp4_comfy_finish_scale(amax.data_ptr(), scale.data_ptr(), _stream(amax)))
    return scale
