"""Autograd wrappers of the fused element-wise kernels (rotary embedding, SwiGLU) used by the decoder workload."""
import torch

from .. import _native as nat


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        # x: [B, S, H, D] BF16 with contiguous (H, D); returns a tensor of the same layout
        b, s, h, d = x.shape
        if x.stride(3) != 1 or x.stride(2) != d or x.stride(0) != s * x.stride(1):
            x = x.contiguous()
        out = torch.empty((b, s, h, d), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            nat.check(nat.lib().nvfp4_rope(x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, h, d, x.stride(1), 0,
                                           nat.stream_of(x)))
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        b, s, h, d = g.shape
        if g.stride(3) != 1 or g.stride(2) != d or g.stride(0) != s * g.stride(1):
            g = g.contiguous()
        out = torch.empty((b, s, h, d), dtype=g.dtype, device=g.device)
        with torch.cuda.device(g.device):
            nat.check(nat.lib().nvfp4_rope(g.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, h, d, g.stride(1), 1,
                                           nat.stream_of(g)))
        return out, None, None


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty_like(gate)
        with torch.cuda.device(gate.device):
            nat.check(nat.lib().nvfp4_swiglu(gate.data_ptr(), up.data_ptr(), None, out.data_ptr(), None, gate.numel(), nat.stream_of(gate)))
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout):
        gate, up = ctx.saved_tensors
        dout = dout.contiguous()
        dgate, dup = torch.empty_like(gate), torch.empty_like(up)
        with torch.cuda.device(gate.device):
            nat.check(nat.lib().nvfp4_swiglu(gate.data_ptr(), up.data_ptr(), dout.data_ptr(), dgate.data_ptr(), dup.data_ptr(), gate.numel(),
                                             nat.stream_of(gate)))
        return dgate, dup


def rope(x, cos, sin):
    """x [B, S, H, D] BF16 -> rotated copy; cos/sin [S, D/2] BF16 contiguous."""
    return _Rope.apply(x, cos, sin)


def swiglu(gate, up):
    return _SwiGLU.apply(gate, up)
