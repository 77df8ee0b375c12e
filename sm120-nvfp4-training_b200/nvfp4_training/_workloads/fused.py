"""Autograd wrappers of the fused BF16 kernels of the decoder workload: residual add + RMSNorm, rotary embedding +
attention over a fused q / k / v projection, SwiGLU over a fused gate / up projection.

Every kernel whose result feeds an NVFP4 layer (in the forward or in the backward pass) also leaves that tensor's amax
on the device; `quant.attach_amax` hands it to the layer's quantiser, which then needs no pass of its own over the tensor.
"""
import torch
from torch.nn import functional as F

from .. import _native as nat
from .._backend import quant as _quant
from .._backend.quant import attach_amax


_SLOTS = {}          # (device index, capturing) -> [zeroed float32 chunk, slots handed out]
_SLOTS_PER_CHUNK = 256


def _amax_slot(device):
    """float32[4] in the layout of nat.amax: [0] receives the amax, the quantiser fills in the scales.  Slots are cut from
    chunks that are zeroed once (one fill kernel per 256 slots instead of one per slot).  A chunk made while a CUDA graph
    is being captured lives in that graph's memory and is zeroed again by every replay; it is never handed out after
    the capture has ended (forget_slots, called where captures begin and end)."""
    key = (torch.device(device).index, torch.cuda.is_current_stream_capturing())
    entry = _SLOTS.get(key)
    if entry is None or entry[1] == _SLOTS_PER_CHUNK:
        entry = _SLOTS[key] = [torch.zeros(4 * _SLOTS_PER_CHUNK, dtype=torch.float32, device=device), 0]
    slot = entry[0][4 * entry[1]: 4 * entry[1] + 4]
    entry[1] += 1
    return slot


def forget_slots():
    _SLOTS.clear()


def _run(fn, *args):
    nat.check(getattr(nat.lib(), fn)(*args))


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, gamma, eps):
        shape = x.shape
        cols = shape[-1]
        x2 = x.reshape(-1, cols)
        d2 = None if delta is None else delta.reshape(-1, cols)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if d2 is not None and not d2.is_contiguous():
            d2 = d2.contiguous()
        rows = x2.shape[0]
        total = torch.empty_like(x2) if d2 is not None else x2
        h = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        amax = _amax_slot(x.device)
        with torch.cuda.device(x.device):
            _run("nvfp4_add_rmsnorm", x2.data_ptr(), nat.ptr(d2), gamma.data_ptr(), float(eps), rows, cols,
                 total.data_ptr() if d2 is not None else None, h.data_ptr(), rstd.data_ptr(), amax.data_ptr(), nat.stream_of(x))
        ctx.save_for_backward(total, rstd, gamma)
        ctx.has_delta, ctx.shape = delta is not None, shape
        ctx.mark_non_differentiable(amax)
        return total.view(shape), h.view(shape), amax

    @staticmethod
    def backward(ctx, dsum, dh, _):
        total, rstd, gamma = ctx.saved_tensors
        rows, cols = total.shape
        if dh is None:
            dh = torch.zeros_like(total)
        dh2 = dh.reshape(rows, cols)
        if not dh2.is_contiguous():
            dh2 = dh2.contiguous()
        dres = None
        if dsum is not None:
            dres = dsum.reshape(rows, cols)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(total)
        dgamma = torch.empty_like(gamma)
        amax = _amax_slot(total.device)
        with torch.cuda.device(total.device):
            parts = int(nat.lib().nvfp4_rmsnorm_bwd_partials(rows, cols))
            partial = torch.empty((parts, cols), dtype=torch.float32, device=total.device)
            _run("nvfp4_rmsnorm_bwd", dh2.data_ptr(), total.data_ptr(), rstd.data_ptr(), gamma.data_ptr(), nat.ptr(dres), rows, cols,
                 dx.data_ptr(), partial.data_ptr(), dgamma.data_ptr(), amax.data_ptr(), nat.stream_of(total))
        dx = attach_amax(dx.view(ctx.shape), amax)
        return dx, (dx if ctx.has_delta else None), dgamma, None


def add_rmsnorm(x, delta, gamma, eps=1e-5):
    """(x + delta, rmsnorm(x + delta) * gamma) for BF16 x, delta (delta may be None) and an FP32 gain; the normalised
    output carries its amax.  In the backward pass the gradient of the sum (which also arrives at `delta`'s producer, an
    NVFP4 layer) carries its amax too."""
    total, h, amax = _AddRMSNorm.apply(x, delta, gamma, eps)
    return total, attach_amax(h, amax)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        shape = gate_up.shape
        width = shape[-1] // 2
        gu = gate_up.reshape(-1, shape[-1])
        if not gu.is_contiguous():
            gu = gu.contiguous()
        rows = gu.shape[0]
        out = torch.empty((rows, width), dtype=gu.dtype, device=gu.device)
        amax = _amax_slot(gu.device)
        with torch.cuda.device(gu.device):
            _run("nvfp4_swiglu", gu.data_ptr(), 2 * width, gu.data_ptr() + 2 * width, 2 * width, None, 0, out.data_ptr(), width, None, 0,
                 rows, width, amax.data_ptr(), nat.stream_of(gu))
        ctx.save_for_backward(gu)
        ctx.shape = shape
        ctx.mark_non_differentiable(amax)
        return out.view(*shape[:-1], width), amax

    @staticmethod
    def backward(ctx, dout, _):
        (gu,) = ctx.saved_tensors
        rows, two = gu.shape
        width = two // 2
        d = dout.reshape(rows, width)
        if not d.is_contiguous():
            d = d.contiguous()
        dgu = torch.empty_like(gu)
        amax = _amax_slot(gu.device)
        with torch.cuda.device(gu.device):
            _run("nvfp4_swiglu", gu.data_ptr(), two, gu.data_ptr() + 2 * width, two, d.data_ptr(), width, dgu.data_ptr(), two,
                 dgu.data_ptr() + 2 * width, two, rows, width, amax.data_ptr(), nat.stream_of(gu))
        return attach_amax(dgu.view(ctx.shape), amax)


def swiglu(gate_up):
    """silu(gate) * up over a fused projection [..., 2 * width] = [gate | up]; result and gradient carry their amax."""
    out, amax = _SwiGLU.apply(gate_up)
    return attach_amax(out, amax)


class _RopeAttention(torch.autograd.Function):
    """Causal attention over a fused projection qkv [B, S, 3 * H * D] = [q | k | v]: q and k are rotated into one buffer by
    a single launch, the attention itself is PyTorch's fused SDPA (BF16, as in the reference's workloads), and the
    backward pass writes the three gradients into one [B, S, 3 * H * D] tensor (inverse rotation of dq and dk, copy of
    dv) together with its amax."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, heads):
        b, s, three = qkv.shape
        width = three // 3
        d = width // heads
        if not qkv.is_contiguous():
            qkv = qkv.contiguous()
        qk = torch.empty((b, s, 2, heads, d), dtype=qkv.dtype, device=qkv.device)
        with torch.cuda.device(qkv.device):
            _run("nvfp4_rope", qkv.data_ptr(), qk.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, 2 * heads, d, three, 2 * width, 0,
                 None, nat.stream_of(qkv))
        v = qkv.view(b, s, 3, heads, d)[:, :, 2]
        with torch.enable_grad():
            leaves = [t.detach().requires_grad_(True) for t in (qk[:, :, 0], qk[:, :, 1], v)]
            out = F.scaled_dot_product_attention(*(t.transpose(1, 2) for t in leaves), is_causal=True)
        ctx.inner, ctx.leaves = out, leaves
        ctx.save_for_backward(cos, sin)
        ctx.dims = (b, s, heads, d)
        return out.detach().transpose(1, 2).reshape(b, s, width)

    @staticmethod
    def backward(ctx, grad):
        cos, sin = ctx.saved_tensors
        b, s, heads, d = ctx.dims
        width = heads * d
        g = grad.view(b, s, heads, d).transpose(1, 2)
        dq, dk, dv = torch.autograd.grad(ctx.inner, ctx.leaves, g)
        ctx.inner = ctx.leaves = None
        dqkv = torch.empty((b, s, 3 * width), dtype=grad.dtype, device=grad.device)
        amax = _amax_slot(grad.device)
        parts = [t if (t.stride(3) == 1 and t.stride(2) == d and t.stride(0) == s * t.stride(1)) else t.contiguous() for t in (dq, dk, dv)]
        with torch.cuda.device(grad.device):
            _run("nvfp4_rope_qkv_bwd", parts[0].data_ptr(), parts[0].stride(1), parts[1].data_ptr(), parts[1].stride(1),
                 parts[2].data_ptr(), parts[2].stride(1), dqkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, heads, d,
                 amax.data_ptr(), nat.stream_of(grad))
        return attach_amax(dqkv, amax), None, None, None


def rope_attention(qkv, cos, sin, heads):
    return _RopeAttention.apply(qkv, cos, sin, heads)


# ---- single-tensor forms kept for models that do not fuse their projections -------------------------------------------
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        b, s, h, d = x.shape
        if x.stride(3) != 1 or x.stride(2) != d or x.stride(0) != s * x.stride(1):
            x = x.contiguous()
        out = torch.empty((b, s, h, d), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            _run("nvfp4_rope", x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, h, d, x.stride(1), h * d, 0, None,
                 nat.stream_of(x))
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        b, s, h, d = g.shape
        if g.stride(3) != 1 or g.stride(2) != d or g.stride(0) != s * g.stride(1):
            g = g.contiguous()
        out = torch.empty((b, s, h, d), dtype=g.dtype, device=g.device)
        amax = _amax_slot(g.device)
        with torch.cuda.device(g.device):
            _run("nvfp4_rope", g.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, h, d, g.stride(1), h * d, 1,
                 amax.data_ptr(), nat.stream_of(g))
        return attach_amax(out, amax), None, None


def rope(x, cos, sin):
    """x [B, S, H, D] BF16 -> rotated copy; cos / sin [S, D / 2] BF16 contiguous."""
    return _Rope.apply(x, cos, sin)


_quant._CAPTURE_EDGE_HOOKS.append(forget_slots)


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows, cols = logits.shape
        lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
        row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        loss = torch.empty((), dtype=torch.float32, device=logits.device)
        with torch.cuda.device(logits.device):
            _run("nvfp4_cross_entropy_fwd", logits.data_ptr(), logits.stride(0), targets.data_ptr(), rows, cols, lse.data_ptr(),
                 row_loss.data_ptr(), loss.data_ptr(), nat.stream_of(logits))
        ctx.save_for_backward(logits, targets, lse)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        logits, targets, lse = ctx.saved_tensors
        rows, cols = logits.shape
        grad_out = grad_out.float().contiguous()
        dlogits = torch.empty((rows, cols), dtype=torch.bfloat16, device=logits.device)
        amax = _amax_slot(logits.device)
        with torch.cuda.device(logits.device):
            _run("nvfp4_cross_entropy_bwd", logits.data_ptr(), logits.stride(0), targets.data_ptr(), lse.data_ptr(), grad_out.data_ptr(),
                 rows, cols, dlogits.data_ptr(), cols, amax.data_ptr(), nat.stream_of(logits))
        return attach_amax(dlogits, amax), None


def cross_entropy(logits, targets):
    """Mean token cross-entropy of BF16 logits [rows, cols] against int64 targets [rows] in two kernels (loss; gradient with
    its amax), or torch's on an FP32 copy where the shape does not fit them."""
    rows, cols = logits.shape
    fits = (logits.is_cuda and logits.dtype == torch.bfloat16 and cols % 8 == 0 and cols <= 32768 and logits.stride(1) == 1
            and logits.stride(0) % 8 == 0 and logits.data_ptr() % 16 == 0 and targets.dtype == torch.int64)
    if not fits:
        return torch.nn.functional.cross_entropy(logits.float(), targets)
    return _CrossEntropy.apply(logits, targets.contiguous())
