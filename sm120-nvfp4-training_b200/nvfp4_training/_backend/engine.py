"""Model conversion: master-weight storage, layer class swap and the matching optimizer.

Semantics of the reference's engine6.configure (src/nvfp4_training/_backend/engine6.py:210-305): validation, direct CPU
conversion, per-layer flags, split / FP8 master initialisation, checkpoint-visible buffers.
"""
from __future__ import annotations

import math
from collections import Counter

import torch
from torch import nn

from .. import _native as nat
from .linear import AutocastLinear, Linear6
from .optimizer import FORMATS, AdamW, AdamW6, cdiv
from .quant import get_signs


def unit_for(p):
    """Power-of-two unit of an FP8 master: the largest weight lands near 48 (master8.py:8-12)."""
    lo, hi = torch.aminmax(p.detach())
    maximum = max(abs(lo.item()), abs(hi.item()))
    if not math.isfinite(maximum):
        raise ValueError('Nonfinite initial weight')
    return 2. ** math.ceil(math.log2(max(maximum, 1e-20) / 48.))


def _load_legacy_unit(module, state, prefix, *args):
    key = prefix + "_v6_unit_buffer"
    unit = state.get(key)
    if unit is not None and unit.ndim == 0 and unit.dtype == torch.float32:
        state[key] = unit.expand_as(module._v6_unit_buffer)


def _convert_layer(layer, remat, fp4):
    if type(layer) is not nn.Linear and not isinstance(layer, Linear6):
        raise TypeError('Custom linear layer')
    if fp4:
        layer.__class__ = Linear6
        layer.register_buffer('_nvfp4_signs', get_signs(layer.weight.device), persistent=False)
        layer._nvfp4_save_packed = True
        p = layer.weight
        p._v4_request_scale = True
        p._v6_fast_scale = True
        p._v6_act_pair = True
        if remat:
            p._v6_remat = True


def configure(model, mode, fmt, *, lr=1e-4, tiles=4, warps=4, prepack=False, pack_warps=8, remat=False, direct=False, mma_k=0,
              mma_warps=8, compact_embedding=False, act_pair=False, fast_scale=False):
    """Set up a fresh contiguous FP32 model (on CPU for direct conversion, else CUDA) for NVFP4 or dense BF16 compute."""
    if mode not in ('bf16', 'fp4') or fmt not in FORMATS:
        raise ValueError('Unknown compute mode or storage format')
    if tiles not in (1, 2, 4, 8, 16) or warps not in (4, 8, 16) or mma_warps not in (4, 8):
        raise ValueError('Unsupported optimizer launch configuration')
    if compact_embedding:
        raise NotImplementedError('compact tied embeddings are not enabled in this interface')
    if prepack and remat:
        raise ValueError('Choose one weight encoding strategy')
    if prepack and FORMATS[fmt][0] == 8:
        raise ValueError('Prepacking is not enabled for FP8 storage')
    if mode == 'bf16':
        raise NotImplementedError("precision='bf16' is the dense control path of the reference; it is not part of the NVFP4 hot path")
    master = FORMATS[fmt][0]
    if direct and master not in (8, 16, 17):
        raise ValueError('Direct CPU conversion requires an FP16, BF16 or FP8 master storage format')
    params = list(model.parameters())
    if any((p.device.type != ('cpu' if direct else 'cuda')) or p.dtype != torch.float32 or not p.is_contiguous() for p in params):
        raise ValueError('Expected a fresh contiguous FP32 model on CPU for direct conversion, or CUDA otherwise')
    if len({p.untyped_storage().data_ptr() for p in params}) != len(params):
        raise ValueError('Distinct parameters must not share storage')
    counts = Counter(id(p) for _, p in model.named_parameters(remove_duplicate=False))

    def narrow(layer):
        return isinstance(layer, nn.Linear) and counts[id(layer.weight)] == 1 and layer.weight.numel() >= 4096

    if master == 8:
        for layer in model.modules():
            if narrow(layer):
                layer.register_buffer('_v6_unit_buffer', torch.tensor(unit_for(layer.weight), device=layer.weight.device, dtype=torch.float32))
    if master == 17:
        bounds = [torch.aminmax(m.weight.detach()) for m in model.modules() if narrow(m)]
        if bounds:
            extrema = torch.stack([v for pair in bounds for v in pair])
            if not ((extrema.abs() <= 65504).all().item()):
                raise ValueError('The initial weight range is not representable in FP16')
    if direct:
        dtype = torch.float16 if master == 17 else torch.bfloat16
        for layer in model.modules():
            if narrow(layer):
                if master == 8:
                    layer.weight.data = (layer.weight.detach() / layer._v6_unit_buffer).to(torch.float8_e4m3fn)
                else:
                    layer.weight.data = layer.weight.detach().to(dtype)
        model.cuda()
        params = list(model.parameters())
        new_counts = Counter(id(p) for _, p in model.named_parameters(remove_duplicate=False))
        if sorted(new_counts.values()) != sorted(counts.values()):
            raise RuntimeError('Device transfer changed parameter sharing')
        counts = new_counts
    for layer in model.modules():
        if isinstance(layer, nn.Linear):
            _convert_layer(layer, remat, True)
    opt = AdamW6(params, fmt, lr=lr, tiles=tiles, warps=warps)
    opt.param_groups[0].update(prepack=prepack, pack_warps=pack_warps, mma_warps=mma_warps)
    for layer in model.modules():
        if not isinstance(layer, nn.Linear):
            continue
        p = layer.weight
        if counts[id(p)] == 1 and p.numel() >= 4096 and not remat:
            p._v6_packable = True        # the optimizer may emit this weight's packings (captured steps with prepack)
        if master != 32 and counts[id(p)] == 1 and p.numel() >= 4096:
            if master == 8:
                if not direct:
                    p.data = (p.detach() / layer._v6_unit_buffer).to(torch.float8_e4m3fn)
                layer._v6_unit_buffer = layer._v6_unit_buffer.expand(cdiv(p.numel(), 512)).clone()
                p._v6_unit = layer._v6_unit_buffer
                layer.register_load_state_dict_pre_hook(_load_legacy_unit)
            elif not direct:
                hi, tail = nat.split_init(p.detach(), master)
                p.data = hi
                if master == 24:
                    opt.state[p]['tail'] = tail
    return model, opt
