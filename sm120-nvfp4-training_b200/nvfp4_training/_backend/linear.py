"""Autograd operator of a converted nn.Linear: three NVFP4 GEMMs per layer and step.

Behaviour follows the reference's _LinearFn6 (src/nvfp4_training/_backend/linear6.py:8-152) and AutocastLinear
(src/nvfp4_training/_linear.py:5-12):
  forward   x -> (row packing, RHT-transposed packing) in one read; weight -> both orientations in one read with the
            tensor scale cached by the optimizer; y = X W^T (+ bias) on the tcgen05 kernel; the packed X^T replaces X
            in the saved state;
  backward  g -> (SR row packing, SR RHT-transposed packing); dX = G W; dW = G^T X either materialised or, when the
            optimizer collects gradients itself, left as the BF16 accumulator image plus the two tensor scales.
"""
from __future__ import annotations

import torch
from torch import nn

from . import quant
from .quant import Packed, dual, matmul, pair, quantize, raw_matmul, round128, single, supported, weight_scale, _STATS


def decoded(w: torch.Tensor) -> torch.Tensor:
    """BF16 image of a master weight; FP8 masters carry a power-of-two unit per 512 weights (master8.py:19-23)."""
    if w.dtype != torch.float8_e4m3fn:
        return w.bfloat16()
    unit = w._v6_unit
    flat = w.detach().reshape(-1).float()
    scale = unit.repeat_interleave(512)[: flat.numel()]
    return (flat * scale).bfloat16().view(w.shape)


def _flat(t: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """2-D view of an activation or gradient; an amax its producer left on the device stays attached to the view."""
    flat = t.reshape(rows, cols)
    if flat is not t:
        hint = quant.known_amax(t)
        if hint is not None and flat.data_ptr() == t.data_ptr():
            quant.attach_amax(flat, hint)
    return flat


def _cached_scale(w: torch.Tensor):
    graph_scale = getattr(w, "_v5_graph_scale", None)
    if graph_scale is not None:
        return graph_scale
    cached = getattr(w, "_v4_scale", None)
    if cached is not None:
        version, ptr, stream, value = cached
        if version == w._version and ptr == w.data_ptr() and stream == torch.cuda.current_stream(w.device).cuda_stream:
            _STATS["optimizer_scale_hits"] += 1
            return value
    return None


def _source(w: torch.Tensor) -> torch.Tensor:
    """What the quantiser reads for a weight: FP32 / FP16 / BF16 masters directly, FP8 masters decoded."""
    return decoded(w) if w.dtype == torch.float8_e4m3fn else w.detach()


def _is_fp8(w: torch.Tensor) -> bool:
    return w.dtype == torch.float8_e4m3fn and w.is_contiguous() and getattr(w, "_v6_unit", None) is not None


def encode(w: torch.Tensor, scale: torch.Tensor, *, row: bool = True, trans: bool = True):
    """FP8 master -> (d, s, scale, dt, st) straight from the E4M3 codes and their per-512 units, no dense copy
    (master8.encode, master8.py:50-56); orientations that are not asked for come back as None."""
    d, s, dt, st = quant.nat.quantize_fp8_weight(w.detach().view(torch.uint8), w._v6_unit, scale, row=row, col=trans)
    return d, s, scale, dt, st


def grad_quant(g, signs, w, rht=False):
    """SR quantisation of a gradient; under graph replay the seed is offset + device base (nvfp4_v5.py:19-32)."""
    clock = getattr(w, "_v5_clock", None)
    if clock is None:
        return quantize(g, signs=signs, sr=True, rht=rht)
    offset = clock.sr_calls
    clock.sr_calls += 1
    return quantize(g, signs=signs, sr=True, rht=rht, seed=offset, base=clock.seed)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, signs, need_x, need_w, need_bias, save_packed):
        original_shape = tuple(x.shape)
        x2 = _flat(x, -1, x.shape[-1])
        m, k = x2.shape
        n = w.shape[0]
        pts = _cached_scale(w)
        use_dual = getattr(w, "_v6_act_pair", False) and need_w and save_packed and supported(x2)
        xp = None
        if use_dual:
            a, xp = dual(x2, signs)
        else:
            a = quantize(x2, signs=signs)
        fp8 = _is_fp8(w)
        contiguous = w.is_contiguous()
        remat = getattr(w, "_v6_remat", False) and contiguous
        paired = not remat and need_x and contiguous
        # FP8 masters are read by the quantiser as they are stored; only a missing tensor scale (the first step of a
        # model, before the optimizer has published one) needs the dense BF16 image
        src = w.detach() if (fp8 and pts is not None) else _source(w)
        if pts is None and (paired or remat):
            pts = weight_scale(src)
        emitted = getattr(w, "_v6_pack", None) if contiguous and not remat and pts is not None else None
        if emitted is not None and emitted["version"] == w._version and emitted["scale"] is pts:
            # the optimizer wrote both packings of this weight, against this scale, in its last update
            data, scale, td, ts = emitted["buffers"]
            b = Packed(data, scale, pts, w.dtype)
            _STATS["quant"] += 2
            _STATS["reused_weight_amax"] += 1
            _STATS["prepacked_weight"] = _STATS.get("prepacked_weight", 0) + 1
        elif paired:
            data, scale, pts, td, ts = encode(w, pts) if fp8 else pair(src, pts)
            b = Packed(data, scale, pts, w.dtype)
            _STATS["quant"] += 2
            _STATS["reused_weight_amax"] += 1
            _STATS["v5_pair"] += 1
        elif remat:
            wd, ws = encode(w, pts, trans=False)[:2] if fp8 else single(src, pts, False)
            b = Packed(wd, ws, pts, w.dtype)
            _STATS["quant"] += 1
        elif fp8 and pts is not None:
            wd, ws = encode(w, pts, trans=False)[:2]
            b = Packed(wd, ws, pts, w.dtype)
            _STATS["quant"] += 1
        else:
            b = quantize(src, signs=signs, pts=pts)
        y = matmul(a, b, rows=m, cols=n, output_dtype=x.dtype, bias=bias)
        tensors = [w, b.pts, signs]
        if need_w:
            if save_packed:
                if xp is None:
                    xp = quantize(x2.t(), rht=True, signs=signs)
                tensors += [xp.data, xp.scale, xp.pts]
                _STATS["packed_activation_saved"] += 1
            else:
                tensors += [x2]
        ctx.paired = paired
        if paired:
            tensors.extend((td, ts))
        ctx.save_for_backward(*tensors)
        ctx.remat, ctx.dual = remat, getattr(w, "_v6_act_pair", False)
        ctx.original_shape, ctx.xdtype = original_shape, x.dtype
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.need_x, ctx.need_w, ctx.need_bias, ctx.save_packed = need_x, need_w, need_bias, save_packed
        ctx.m, ctx.k, ctx.n = m, k, n
        return y.reshape(*original_shape[:-1], n)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        saved = ctx.saved_tensors
        w, wpts, signs = saved[:3]
        g = _flat(grad, ctx.m, ctx.n)
        if any(s == 0 for s in g.stride()):
            g = g.contiguous()
        dx = dw = db = None
        ahead = adjoint = None
        if ctx.dual and ctx.need_x and ctx.need_w and supported(g):
            ahead, adjoint = dual(g, signs, sr=True, clock=getattr(w, "_v5_clock", None))
        if ctx.need_x:
            aq = ahead if ahead is not None else grad_quant(g, signs, w)
            if ctx.remat:
                wd, ws = encode(w, wpts, row=False)[3:] if _is_fp8(w) else single(_source(w), wpts, True)
                wq = Packed(wd, ws, wpts, w.dtype)
                _STATS["quant"] += 1
            elif ctx.paired:
                wq = Packed(saved[-2], saved[-1], wpts, w.dtype)
            elif _is_fp8(w):
                wd, ws = encode(w, wpts, row=False)[3:]
                wq = Packed(wd, ws, wpts, w.dtype)
                _STATS["quant"] += 1
            else:
                wq = quantize(_source(w).t(), signs=signs, pts=wpts)
            dx = matmul(aq, wq, rows=ctx.m, cols=ctx.k, output_dtype=ctx.xdtype)
            dx = dx.reshape(ctx.original_shape)
        if ctx.need_w:
            aq = adjoint if adjoint is not None else grad_quant(g.t(), signs, w, rht=True)
            if ctx.save_packed:
                xq = Packed(saved[3], saved[4], saved[5], ctx.xdtype)
            else:
                xq = quantize(saved[3].t(), rht=True, signs=signs)
            sink = getattr(w, "_v4_pending", None)
            if w.dtype == torch.float8_e4m3fn and (sink is None or w in sink or aq.dtype != torch.bfloat16):
                raise RuntimeError("FP8 master requires BF16 activations and a single deferred dW contribution")
            reducer = getattr(w, "_dp_reducer", None)
            if reducer is not None and sink is not None and w not in sink:
                # data parallel: the scaled BF16 gradient goes straight into this parameter's bucket slot
                slot = reducer.slot(w)
                quant.nat.gemm(aq.data, aq.scale, aq.pts, xq.data, xq.scale, xq.pts, rows=ctx.n, cols=ctx.k,
                               out_dtype=torch.bfloat16, raw_bf16=True, out=slot.view(ctx.n, ctx.k))
                _STATS["fp4_gemm"] += 1
                sink[w] = (slot, None, None)
                reducer.ready(w)
            elif sink is None or w in sink or aq.dtype != torch.bfloat16:
                dw = matmul(aq, xq, rows=ctx.n, cols=ctx.k, output_dtype=torch.bfloat16 if w.dtype == torch.float16 else
                            (w.dtype if w.dtype in (torch.float32, torch.bfloat16) else torch.bfloat16))
            else:
                sink[w] = (raw_matmul(aq, xq, ctx.n, ctx.k), aq.pts, xq.pts)
        if ctx.need_bias:
            db = g.sum(0).to(ctx.bias_dtype)
        return dx, dw, db, None, None, None, None, None


class Linear6(nn.Linear):
    """nn.Linear whose three GEMMs run in NVFP4; parameters stay the module's own Parameter objects."""

    def forward(self, x):
        if x.device != self.weight.device or x.shape[-1] != self.in_features:
            raise ValueError("Invalid activation device or features")
        active = torch.is_grad_enabled()
        return _LinearFn.apply(x, self.weight, self.bias, self._nvfp4_signs,
                               active and x.requires_grad, active and self.weight.requires_grad,
                               active and self.bias is not None and self.bias.requires_grad, self._nvfp4_save_packed)


class AutocastLinear(Linear6):
    """Honours BF16 autocast at the NVFP4 boundary, including FP32 norm / embedding outputs."""

    def forward(self, input):
        if input.dtype != torch.bfloat16:
            if (input.dtype not in (torch.float32, torch.float16) or not torch.is_autocast_enabled("cuda")
                    or torch.get_autocast_dtype("cuda") != torch.bfloat16):
                raise TypeError("NVFP4 Linear expects BF16 activations or CUDA BF16 autocast.")
            input = input.to(torch.bfloat16)
        return super().forward(input)
