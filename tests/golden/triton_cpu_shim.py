"""Make the Triton CPU interpreter faithful enough to execute the reference's Triton kernels.

Used only by ``make_golden.py`` (fixture generation, run once in the build container where the
reference sources are mounted).  Two gaps of ``TRITON_INTERPRET=1`` are closed:

* float down-casts: the stock interpreter truncates mantissas; the GPU the kernels were written for
  rounds to nearest even (PTX ``cvt.rn``).  Casts to bf16 / fp16 / fp8e4nv are redirected to
  PyTorch's CPU conversions, which implement IEEE round-to-nearest-even (and E4M3 saturating
  semantics identical to ``cvt.rn.satfinite`` inside the finite range the kernels use).
* scalar arguments: the compiled launcher passes a Python float as an FP32 kernel parameter, so
  expressions such as ``1. - b1`` are FP32 device arithmetic; the stock interpreter keeps the Python
  double.  Float arguments are turned into FP32 scalars here.
* inline PTX: the three instructions the reference embeds are given their PTX-ISA meaning:
  ``mul.rn.f32`` (one rounded multiply), ``cvt.rni.s32.f32`` (round half to even to int32) and
  ``cvt.rn.satfinite.e2m1x2.f32`` (two floats to two e2m1 nibbles, nearest, ties to even code,
  first source operand in the high nibble).
"""
import os

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import triton.language as tl
from triton.runtime import interpreter as _interp

_orig_convert = _interp._convert_float
_TORCH = {tl.bfloat16: torch.bfloat16, tl.float16: torch.float16, tl.float8e4nv: torch.float8_e4m3fn}
_VIEW = {tl.bfloat16: torch.int16, tl.float16: torch.int16, tl.float8e4nv: torch.uint8}
_NPVIEW = {tl.bfloat16: np.uint16, tl.float16: np.uint16, tl.float8e4nv: np.uint8}


def _as_f32(data, dtype):
    if dtype == tl.float32:
        return torch.from_numpy(np.ascontiguousarray(data).view(np.float32).copy())
    if dtype == tl.float64:
        return torch.from_numpy(np.ascontiguousarray(data).view(np.float64).copy())
    raw = np.ascontiguousarray(data).view(_NPVIEW[dtype]).copy()
    if dtype == tl.float8e4nv:
        return torch.from_numpy(raw).view(torch.float8_e4m3fn).float()
    return torch.from_numpy(raw.view(np.int16)).view(_TORCH[dtype]).float()


def _convert_float(input, input_dtype, output_dtype, rounding_mode):
    known = (tl.float32, tl.float64, tl.bfloat16, tl.float16, tl.float8e4nv)
    if input_dtype not in known or output_dtype not in known:
        return _orig_convert(input, input_dtype, output_dtype, rounding_mode)
    shape = input.shape
    value = _as_f32(input, input_dtype)
    if output_dtype == tl.float32:
        return value.float().numpy().reshape(shape).view(np.uint32)
    if output_dtype == tl.float64:
        return value.double().numpy().reshape(shape).view(np.uint64)
    if output_dtype == tl.float8e4nv:
        v32 = value.float()
        out = v32.to(torch.float8_e4m3fn).view(torch.uint8)
        # round_e4m3 in master8.py relies on "NaN in, NaN code out"; torch agrees.
        return out.numpy().reshape(shape)
    out = value.float().to(_TORCH[output_dtype]).view(torch.int16).numpy().view(np.uint16)
    return out.reshape(shape)


_interp._convert_float = _convert_float


def _e2m1_rne(v):
    a = np.abs(v)
    c = np.zeros(v.shape, np.int32)
    c = np.where(a > 0.25, 1, c)
    c = np.where(a >= 0.75, 2, c)
    c = np.where(a > 1.25, 3, c)
    c = np.where(a >= 1.75, 4, c)
    c = np.where(a > 2.5, 5, c)
    c = np.where(a >= 3.5, 6, c)
    c = np.where(a > 5.0, 7, c)
    return c | np.where(np.signbit(v), 8, 0)


class _AsmCall:
    def __init__(self, handle):
        self._handle = handle

    def get_result(self, index):
        assert index == 0
        return self._handle


def _inline_asm(self, inlineAsm, constraints, values, type, isPure, pack):
    args = [np.asarray(v.data) for v in values]
    shape = np.broadcast_shapes(*[a.shape for a in args])
    args = [np.broadcast_to(a, shape) for a in args]
    if "mul.rn.f32" in inlineAsm:
        out = (args[0].astype(np.float32) * args[1].astype(np.float32)).astype(np.float32)
        return _AsmCall(_interp.TensorHandle(out, tl.float32))
    if "cvt.rni.s32.f32" in inlineAsm:
        return _AsmCall(_interp.TensorHandle(np.rint(args[0].astype(np.float32)).astype(np.int32), tl.int32))
    if "cvt.rn.satfinite.e2m1x2.f32" in inlineAsm:
        # asm text: "cvt... byte,$2,$1" with args [lo, hi]  ->  d = {e2m1(hi) << 4 | e2m1(lo)}
        lo, hi = args[0].astype(np.float32), args[1].astype(np.float32)
        return _AsmCall(_interp.TensorHandle((_e2m1_rne(lo) | (_e2m1_rne(hi) << 4)).astype(np.int32), tl.int32))
    raise NotImplementedError(inlineAsm)


_interp.InterpreterBuilder.create_inline_asm = _inline_asm


_orig_implicit_cvt = _interp._implicit_cvt


def _implicit_cvt(arg):
    if isinstance(arg, float):
        return tl.tensor(_interp.TensorHandle(np.array([arg], dtype=np.float32), tl.float32), tl.float32)
    return _orig_implicit_cvt(arg)


_interp._implicit_cvt = _implicit_cvt
