"""Frozen Linear over an NVFP4 checkpoint kept exactly as stored, with native input gradients.

Interface and behaviour of the reference's PackedNVFP4Linear (src/precision_lora/packed.py:36-152; same constructor,
buffers, attribute names and error messages, which its state dicts and callers depend on): the source nibbles (even
element in the high nibble) and swizzled E4M3 scales are preserved; nothing is inferred from names and no floating-point
weight is quantised implicitly.  Forward quantises the activation (RNE, no rotation) and multiplies by the stored
packing; backward quantises the gradient with the H128 rotation and stochastic rounding and multiplies by the rotated
transpose of the weight, which is either rebuilt from the packed bytes on every backward (backward_mode='recompute') or
kept on the device ('cache').  Both modes produce identical values.

The file is organised in three parts: `_Stored` checks a checkpoint's tensors and brings them to the kernels' 128-aligned
geometry, `PackedNVFP4Linear` holds the resulting buffers, and the two products (forward, input gradient) are separate
methods over the kernels of _packed_cuda.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn
from torch.nn import functional as F

LAYOUT = "comfy-high-first-swizzle128x4"
_MAGNITUDE_BITS = 0x77       # both nibbles without their sign bits: zero iff both elements decode to (+-)0


def _round128(n):
    return (n + 127) // 128 * 128


def _scale_positions(rows, groups, width, device):
    """Flat position of scale byte (row, group) in the 128 x 4 swizzle of a tensor `width` columns wide."""
    r = torch.arange(rows, device=device)[:, None]
    g = torch.arange(groups, device=device)[None, :]
    per_row_block = (width + 63) // 64
    return (r // 128) * per_row_block * 512 + (g // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + g % 4


def _fail_unless(ok, error, message):
    if not ok:
        raise error(message)


@dataclass
class _Stored:
    """A checkpoint weight after validation: 128-aligned payload and scales, logical shape."""
    payload: torch.Tensor
    scales: torch.Tensor
    out_features: int
    in_features: int

    @classmethod
    def accept(cls, packed, block_scale, tensor_scale, shape, bias, input_scale):
        _fail_unless(packed.ndim == 2 and packed.dtype == torch.uint8 and packed.is_cuda, TypeError,
                     "packed must be a CUDA uint8 [rows, cols/2] tensor")
        _fail_unless(block_scale.dtype == torch.float8_e4m3fn and tensor_scale.dtype == torch.float32 and tensor_scale.numel() == 1,
                     TypeError, "Expected E4M3 block scales and one FP32 tensor scale")
        tensors = [packed, block_scale, tensor_scale, *(t for t in (bias, input_scale) if t is not None)]
        _fail_unless(all(t.device == packed.device and not t.requires_grad for t in tensors), ValueError,
                     "Base tensors must be frozen and on the same CUDA device")
        rows, width = packed.shape[0], packed.shape[1] * 2
        _fail_unless(rows >= 1 and width >= 16 and width % 16 == 0, ValueError, "Stored width must contain complete 16-value scale blocks")
        n, k = (rows, width) if shape is None else tuple(shape)
        _fail_unless(type(n) is int and type(k) is int and 0 < n <= rows and 0 < k <= width, ValueError, "Invalid logical shape")
        _fail_unless(block_scale.numel() == _round128(rows) * ((width + 63) // 64) * 4, ValueError,
                     "Swizzled scale storage size does not match the packed shape")
        _fail_unless(bool(torch.isfinite(tensor_scale).all()) and tensor_scale.item() > 0, ValueError,
                     "Tensor scale must be finite and positive")
        _fail_unless(bias is None or (bias.shape == (n,) and bias.is_floating_point()), ValueError, "Bias must have logical output width")
        _fail_unless(input_scale is None or (input_scale.shape == (k,) and bool(torch.isfinite(input_scale).all())), ValueError,
                     "AWQ input_scale must be a finite vector of logical input width")
        # the padding has to decode to zero: the rotation of the backward operand would spread anything else over 128 rows
        _fail_unless(n == rows or not (packed[n:] & _MAGNITUDE_BITS).any(), ValueError, "Nonzero row padding in source weights")
        if k < width:
            beyond = (packed[:n, (k + 1) // 2:] & _MAGNITUDE_BITS).any()
            shared_byte = k % 2 and (packed[:n, k // 2] & 0x07).any()       # odd k: the low nibble of the last byte is padding
            _fail_unless(not (beyond or shared_byte), ValueError, "Nonzero column padding in source weights")
        device = packed.device
        raw_scales = block_scale.contiguous().view(torch.uint8).flatten()
        live = raw_scales[_scale_positions(rows, width // 16, width, device)]
        healthy = not (live & 0x80).any() and bool(torch.isfinite(live.view(torch.float8_e4m3fn).float()).all())
        _fail_unless(healthy, ValueError, "Block scales must be finite and nonnegative")
        rows_p, width_p = _round128(rows), _round128(width)
        if (rows_p, width_p) == (rows, width):
            return cls(packed.contiguous(), block_scale.contiguous(), n, k)
        payload = F.pad(packed, (0, (width_p - width) // 2, 0, rows_p - rows)).contiguous()
        placed = torch.zeros(rows_p * width_p // 16, dtype=torch.uint8, device=device)      # padding blocks: scale code 0
        placed[_scale_positions(rows, width // 16, width_p, device)] = live
        return cls(payload, placed.view(torch.float8_e4m3fn), n, k)


class _BaseFunction(torch.autograd.Function):
    """The packed layer used on its own (without an adapter): forward product and native input gradient."""

    @staticmethod
    def forward(ctx, x, base):
        kind = x.device.type
        compute = torch.get_autocast_dtype(kind) if torch.is_autocast_enabled(kind) else x.dtype
        ctx.base, ctx.x_shape, ctx.x_dtype = base, x.shape, x.dtype
        y = base.multiply(x.reshape(-1, x.shape[-1]).to(compute))
        return y.reshape(*x.shape[:-1], base.out_features)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        dx = ctx.base.multiply(grad.reshape(-1, grad.shape[-1]), backward=True)
        return dx.reshape(ctx.x_shape).to(ctx.x_dtype), None


class PackedNVFP4Linear(nn.Module):
    """Frozen Linear for high-nibble-first E2M1 payloads with 128 x 4 swizzled E4M3 block scales.

    `shape` is the logical (out_features, in_features) before zero padding.  Bias and an optional AWQ `input_scale`
    stay frozen; the input scaling is part of the input gradient.  `seed` fixes the rotation signs and the start of
    the stochastic-rounding counter."""

    def __init__(self, packed, block_scale, tensor_scale, *, shape=None, bias=None, input_scale=None, layout,
                 backward_mode="recompute", seed=0):
        super().__init__()
        _fail_unless(layout == LAYOUT, ValueError, "Declare layout='comfy-high-first-swizzle128x4'; other layouts need conversion")
        _fail_unless(backward_mode in ("recompute", "cache"), ValueError, "backward_mode must be 'recompute' or 'cache'")
        stored = _Stored.accept(packed, block_scale, tensor_scale, shape, bias, input_scale)
        self.in_features, self.out_features = stored.in_features, stored.out_features
        self.backward_mode, self.layout, self.source_dtype = backward_mode, layout, torch.bfloat16
        device = stored.payload.device
        self.rht_seed = int(seed) % (2 ** 63)
        signs = torch.randint(0, 2, (128,), generator=torch.Generator().manual_seed(self.rht_seed)) * 2 - 1
        for name, value in (("packed", stored.payload), ("block_scale", stored.scales), ("tensor_scale", tensor_scale.reshape(())),
                            ("bias", bias), ("input_scale", input_scale), ("signs", signs.float().to(device)),
                            ("sr_seed", torch.tensor(int(seed) & 0x7fffffff, device=device, dtype=torch.int32))):
            self.register_buffer(name, value)
        from . import _packed_cuda as kernels
        with torch.cuda.device(device):
            self.register_buffer("backward_scale", kernels.backward_scale(self.quant, self.signs))
            kept = kernels.transpose_rht_quant(self.quant, self.signs, self.backward_scale)[:2] if backward_mode == "cache" else (None, None)
        self.register_buffer("backward_packed", kept[0])
        self.register_buffer("backward_blocks", kept[1])

    @property
    def quant(self):
        return self.packed, self.block_scale, self.tensor_scale

    @property
    def device(self):
        return self.packed.device

    # ---- the two products -------------------------------------------------------------------------------------------
    def _check_call(self, x, logical):
        fp32 = (self.tensor_scale, self.backward_scale, self.signs)
        intact = (self.packed.dtype == torch.uint8 and self.block_scale.dtype == torch.float8_e4m3fn
                  and all(t.dtype == torch.float32 for t in fp32) and self.sr_seed.dtype == torch.int32)
        _fail_unless(intact, TypeError, "Packed weight/scale dtypes changed; move the base by device only and use BF16 autocast")
        _fail_unless(x.dtype == torch.bfloat16 and x.device == self.device and x.ndim == 2, TypeError,
                     "Packed NVFP4 GEMMs require BF16 inputs on the base CUDA device")
        _fail_unless(not torch.cuda.is_current_stream_capturing(), RuntimeError,
                     "Packed NVFP4 CUDA graph replay has not been validated; use ordinary eager training")
        _fail_unless(x.shape[-1] == logical, ValueError, "Input width does not match the frozen projection")

    @staticmethod
    def _widen(x, stored_width):
        return x.contiguous() if x.shape[-1] == stored_width else F.pad(x, (0, stored_width - x.shape[-1])).contiguous()

    def _forward_product(self, x, kernels):
        if self.input_scale is not None:
            x = (x * self.input_scale).to(x.dtype)
        act = kernels.quantize(self._widen(x, self.packed.shape[1] * 2))
        y = kernels.matmul(act, self.quant, rows=len(x), cols=self.out_features)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def _input_gradient(self, g, kernels):
        weight = ((self.backward_packed, self.backward_blocks, self.backward_scale) if self.backward_mode == "cache"
                  else kernels.transpose_rht_quant(self.quant, self.signs, self.backward_scale))
        act = kernels.quantize(self._widen(g, self.packed.shape[0]), self.signs, seed=self.sr_seed, sr=True)
        self.sr_seed.add_(1)
        dx = kernels.matmul(act, weight, rows=len(g), cols=self.in_features)
        return dx if self.input_scale is None else (dx * self.input_scale).to(g.dtype)

    def multiply(self, x, backward=False):
        """x @ W^T + bias on the logical shapes, or for backward g @ W; BF16 in, BF16 out."""
        from . import _packed_cuda as kernels
        self._check_call(x, self.out_features if backward else self.in_features)
        with torch.cuda.device(x.device):
            return self._input_gradient(x, kernels) if backward else self._forward_product(x, kernels)

    def forward(self, x):
        return _BaseFunction.apply(x, self)
