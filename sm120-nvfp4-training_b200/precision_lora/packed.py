"""Frozen Linear over an NVFP4 checkpoint kept exactly as stored, with native input gradients.

Interface and behaviour of the reference's PackedNVFP4Linear (src/precision_lora/packed.py:36-152): the source nibbles
(even element in the high nibble) and swizzled E4M3 scales are preserved; nothing is inferred from names and no
floating-point weight is quantised implicitly.  Forward quantises the activation (RNE, no rotation) and multiplies by
the stored packing; backward quantises the gradient with the H128 rotation and stochastic rounding and multiplies by
the rotated transpose of the weight, which is either rebuilt from the packed bytes on every backward
(backward_mode='recompute') or kept on the device ('cache').  Both modes produce identical values.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

LAYOUT = "comfy-high-first-swizzle128x4"


def _round128(n):
    return (n + 127) // 128 * 128


def _indices(rows, groups, width, device):
    """Flat position of scale byte (row, group) in the 128 x 4 swizzle of a tensor `width` columns wide."""
    r = torch.arange(rows, device=device)[:, None]
    b = torch.arange(groups, device=device)[None, :]
    blocks_per_row = (width + 63) // 64
    return (r // 128) * blocks_per_row * 512 + (b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4


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
        if layout != LAYOUT:
            raise ValueError("Declare layout='comfy-high-first-swizzle128x4'; other layouts need conversion")
        if backward_mode not in ("recompute", "cache"):
            raise ValueError("backward_mode must be 'recompute' or 'cache'")
        if packed.ndim != 2 or packed.dtype != torch.uint8 or not packed.is_cuda:
            raise TypeError("packed must be a CUDA uint8 [rows, cols/2] tensor")
        if block_scale.dtype != torch.float8_e4m3fn or tensor_scale.dtype != torch.float32 or tensor_scale.numel() != 1:
            raise TypeError("Expected E4M3 block scales and one FP32 tensor scale")
        given = [packed, block_scale, tensor_scale] + [t for t in (bias, input_scale) if t is not None]
        if any(t.device != packed.device or t.requires_grad for t in given):
            raise ValueError("Base tensors must be frozen and on the same CUDA device")
        rows, width = packed.shape[0], packed.shape[1] * 2
        if rows < 1 or width < 16 or width % 16:
            raise ValueError("Stored width must contain complete 16-value scale blocks")
        n, k = (rows, width) if shape is None else tuple(shape)
        if type(n) is not int or type(k) is not int or not (0 < n <= rows and 0 < k <= width):
            raise ValueError("Invalid logical shape")
        if block_scale.numel() != _round128(rows) * ((width + 63) // 64) * 4:
            raise ValueError("Swizzled scale storage size does not match the packed shape")
        if not torch.isfinite(tensor_scale).all() or tensor_scale.item() <= 0:
            raise ValueError("Tensor scale must be finite and positive")
        if bias is not None and (bias.shape != (n,) or not bias.is_floating_point()):
            raise ValueError("Bias must have logical output width")
        if input_scale is not None and (input_scale.shape != (k,) or not torch.isfinite(input_scale).all()):
            raise ValueError("AWQ input_scale must be a finite vector of logical input width")
        # padding has to decode to zero: the rotation of the backward operand would spread anything else
        magnitude = 0x77
        if n < rows and (packed[n:] & magnitude).any():
            raise ValueError("Nonzero row padding in source weights")
        if k < width:
            odd_tail = k % 2 and (packed[:n, k // 2] & 0x07).any()
            if (packed[:n, (k + 1) // 2:] & magnitude).any() or odd_tail:
                raise ValueError("Nonzero column padding in source weights")
        self.in_features, self.out_features = k, n
        self.backward_mode, self.layout = backward_mode, layout
        self.source_dtype = torch.bfloat16
        rows_p, width_p = _round128(rows), _round128(width)
        exact = (rows_p, width_p) == (rows, width)
        payload = packed.contiguous() if exact else F.pad(packed, (0, (width_p - width) // 2, 0, rows_p - rows)).contiguous()
        stored = block_scale.contiguous().view(torch.uint8).flatten()
        live = stored[_indices(rows, width // 16, width, payload.device)]
        if (live & 0x80).any() or not torch.isfinite(live.view(torch.float8_e4m3fn).float()).all():
            raise ValueError("Block scales must be finite and nonnegative")
        if exact:
            scales = block_scale.contiguous()
        else:   # re-place the live scale bytes for the padded width; padding blocks are zero
            moved = torch.zeros(rows_p * width_p // 16, dtype=torch.uint8, device=payload.device)
            moved[_indices(rows, width // 16, width_p, payload.device)] = live
            scales = moved.view(torch.float8_e4m3fn)
        self.register_buffer("packed", payload)
        self.register_buffer("block_scale", scales)
        self.register_buffer("tensor_scale", tensor_scale.reshape(()))
        self.register_buffer("bias", bias)
        self.register_buffer("input_scale", input_scale)
        self.rht_seed = int(seed) % (2 ** 63)
        generator = torch.Generator().manual_seed(self.rht_seed)
        self.register_buffer("signs", (torch.randint(0, 2, (128,), generator=generator) * 2 - 1).float().to(payload.device))
        self.register_buffer("sr_seed", torch.tensor(int(seed) & 0x7fffffff, device=payload.device, dtype=torch.int32))
        from . import _packed_cuda as cuda
        with torch.cuda.device(payload.device):
            self.register_buffer("backward_scale", cuda.backward_scale(self.quant, self.signs))
            cached = (cuda.transpose_rht_quant(self.quant, self.signs, self.backward_scale) if backward_mode == "cache"
                      else (None, None, None))
        self.register_buffer("backward_packed", cached[0])
        self.register_buffer("backward_blocks", cached[1])

    @property
    def quant(self):
        return self.packed, self.block_scale, self.tensor_scale

    @property
    def device(self):
        return self.packed.device

    def _backward_operand(self):
        if self.backward_mode == "cache":
            return self.backward_packed, self.backward_blocks, self.backward_scale
        from . import _packed_cuda as cuda
        return cuda.transpose_rht_quant(self.quant, self.signs, self.backward_scale)

    def multiply(self, x, backward=False):
        """x @ W^T + bias on the logical shapes, or for backward g @ W; BF16 in, BF16 out."""
        from . import _packed_cuda as cuda
        if (self.packed.dtype != torch.uint8 or self.block_scale.dtype != torch.float8_e4m3fn
                or any(t.dtype != torch.float32 for t in (self.tensor_scale, self.backward_scale, self.signs))
                or self.sr_seed.dtype != torch.int32):
            raise TypeError("Packed weight/scale dtypes changed; move the base by device only and use BF16 autocast")
        if x.dtype != torch.bfloat16 or x.device != self.device or x.ndim != 2:
            raise TypeError("Packed NVFP4 GEMMs require BF16 inputs on the base CUDA device")
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Packed NVFP4 CUDA graph replay has not been validated; use ordinary eager training")
        logical = self.out_features if backward else self.in_features
        if x.shape[-1] != logical:
            raise ValueError("Input width does not match the frozen projection")
        if not backward and self.input_scale is not None:
            x = (x * self.input_scale).to(x.dtype)
        stored = self.packed.shape[0] if backward else self.packed.shape[1] * 2
        v = x.contiguous() if stored == logical else F.pad(x, (0, stored - logical)).contiguous()
        with torch.cuda.device(x.device):
            if backward:
                weight = self._backward_operand()
                act = cuda.quantize(v, self.signs, seed=self.sr_seed, sr=True)
                self.sr_seed.add_(1)
                y = cuda.matmul(act, weight, rows=len(x), cols=self.in_features)
                if self.input_scale is not None:
                    y = (y * self.input_scale).to(x.dtype)
            else:
                y = cuda.matmul(cuda.quantize(v), self.quant, rows=len(x), cols=self.out_features)
                if self.bias is not None:
                    y = y + self.bias.to(y.dtype)
        return y

    def forward(self, x):
        return _BaseFunction.apply(x, self)
