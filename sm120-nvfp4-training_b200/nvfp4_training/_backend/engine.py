"""Model conversion: master-weight storage, layer class swap and the matching optimizer.

`configure` keeps the signature, the checks and the checkpoint-visible results of the reference's engine6.configure
(src/nvfp4_training/_backend/engine6.py:210-305): which weights become narrow masters (a Linear's own weight of at least
4096 elements), the per-512 power-of-two units of FP8 masters and their module buffer, the split BF16 + int8 tail, direct
conversion on the host.  It is organised as a plan (which layer gets which storage) followed by the steps that carry the
plan out.
"""
from __future__ import annotations

import math
from collections import Counter
from dataclasses import dataclass

import torch
from torch import nn

from .. import _native as nat
from .linear import AutocastLinear, Linear6
from .optimizer import FORMATS, AdamW, AdamW6, cdiv
from .quant import get_signs

NARROW_FROM = 4096          # weights below this many elements keep FP32 masters and FP32 moments
UNIT_BLOCK = 512            # weights per power-of-two unit of an FP8 master


def unit_for(p):
    """Power-of-two unit of an FP8 master: the largest weight lands near 48 (master8.py:8-12)."""
    lo, hi = torch.aminmax(p.detach())
    maximum = max(abs(lo.item()), abs(hi.item()))
    if not math.isfinite(maximum):
        raise ValueError('Nonfinite initial weight')
    return 2. ** math.ceil(math.log2(max(maximum, 1e-20) / 48.))


def _load_legacy_unit(module, state, prefix, *args):
    """Checkpoints written when an FP8 master had one scalar unit: spread it over the blocks."""
    key = prefix + "_v6_unit_buffer"
    unit = state.get(key)
    if unit is not None and unit.ndim == 0 and unit.dtype == torch.float32:
        state[key] = unit.expand_as(module._v6_unit_buffer)


@dataclass
class _Plan:
    master: int
    direct: bool
    remat: bool
    narrow: list          # Linear layers whose weight gets the format's narrow master


def _check_request(model, mode, fmt, tiles, warps, mma_warps, prepack, remat, direct, compact_embedding):
    if mode not in ('bf16', 'fp4') or fmt not in FORMATS:
        raise ValueError('Unknown compute mode or storage format')
    if tiles not in (1, 2, 4, 8, 16) or warps not in (4, 8, 16) or mma_warps not in (4, 8):
        raise ValueError('Unsupported optimizer launch configuration')
    if compact_embedding:
        raise NotImplementedError('compact tied embeddings are not enabled in this interface')
    if prepack and remat:
        raise ValueError('Choose one weight encoding strategy')
    master = FORMATS[fmt][0]
    if prepack and master == 8:
        raise ValueError('Prepacking is not enabled for FP8 storage')
    if mode == 'bf16':
        raise NotImplementedError("precision='bf16' is the dense control path of the reference; it is not part of the NVFP4 hot path")
    if direct and master not in (8, 16, 17):
        raise ValueError('Direct CPU conversion requires an FP16, BF16 or FP8 master storage format')
    params = list(model.parameters())
    home = 'cpu' if direct else 'cuda'
    if any(p.device.type != home or p.dtype != torch.float32 or not p.is_contiguous() for p in params):
        raise ValueError('Expected a fresh contiguous FP32 model on CPU for direct conversion, or CUDA otherwise')
    if len({p.untyped_storage().data_ptr() for p in params}) != len(params):
        raise ValueError('Distinct parameters must not share storage')
    return master


def _uses(model):
    """How many times each Parameter object is registered (a head tied to an embedding counts twice)."""
    return Counter(id(p) for _, p in model.named_parameters(remove_duplicate=False))


def _narrow_layers(model, master):
    uses = _uses(model)
    if master == 32:
        return []
    return [m for m in model.modules() if isinstance(m, nn.Linear) and uses[id(m.weight)] == 1 and m.weight.numel() >= NARROW_FROM]


def _convert_on_host(model, plan):
    """Direct conversion: narrow the masters while the model is still on the CPU, then move it; only 1 or 2 bytes per
    weight ever reach the GPU."""
    before = sorted(_uses(model).values())
    for layer in plan.narrow:
        w = layer.weight.detach()
        if plan.master == 8:
            layer.weight.data = (w / layer._v6_unit_buffer).to(torch.float8_e4m3fn)
        else:
            layer.weight.data = w.to(torch.float16 if plan.master == 17 else torch.bfloat16)
    model.cuda()
    if sorted(_uses(model).values()) != before:
        raise RuntimeError('Device transfer changed parameter sharing')


def _attach_nvfp4(layer, remat):
    if type(layer) is not nn.Linear and not isinstance(layer, Linear6):
        raise TypeError('Custom linear layer')
    layer.__class__ = Linear6
    layer.register_buffer('_nvfp4_signs', get_signs(layer.weight.device), persistent=False)
    layer._nvfp4_save_packed = True
    w = layer.weight
    w._v4_request_scale = w._v6_fast_scale = w._v6_act_pair = True
    if remat:
        w._v6_remat = True


def _narrow_on_device(layer, plan, opt):
    """The master storage of one layer (device conversion) and, for FP8, its checkpoint-visible unit vector."""
    p = layer.weight
    if plan.master == 8:
        if not plan.direct:
            p.data = (p.detach() / layer._v6_unit_buffer).to(torch.float8_e4m3fn)
        layer._v6_unit_buffer = layer._v6_unit_buffer.expand(cdiv(p.numel(), UNIT_BLOCK)).clone()
        p._v6_unit = layer._v6_unit_buffer
        layer.register_load_state_dict_pre_hook(_load_legacy_unit)
    elif not plan.direct:
        head, tail = nat.split_init(p.detach(), plan.master)
        p.data = head
        if plan.master == 24:
            opt.state[p]['tail'] = tail


def configure(model, mode, fmt, *, lr=1e-4, tiles=4, warps=4, prepack=False, pack_warps=8, remat=False, direct=False, mma_k=0,
              mma_warps=8, compact_embedding=False, act_pair=False, fast_scale=False):
    """Set up a fresh contiguous FP32 model (on CPU for direct conversion, else CUDA) for NVFP4 compute."""
    master = _check_request(model, mode, fmt, tiles, warps, mma_warps, prepack, remat, direct, compact_embedding)
    plan = _Plan(master, direct, remat, _narrow_layers(model, master))
    if master == 8:
        for layer in plan.narrow:
            unit = torch.tensor(unit_for(layer.weight), device=layer.weight.device, dtype=torch.float32)
            layer.register_buffer('_v6_unit_buffer', unit)
    if master == 17 and plan.narrow:
        bounds = torch.stack([v for layer in plan.narrow for v in torch.aminmax(layer.weight.detach())])
        if not (bounds.abs() <= 65504).all().item():
            raise ValueError('The initial weight range is not representable in FP16')
    if direct:
        _convert_on_host(model, plan)
    uses = _uses(model)
    for layer in model.modules():
        if isinstance(layer, nn.Linear):
            _attach_nvfp4(layer, remat)
            p = layer.weight
            if uses[id(p)] == 1 and p.numel() >= NARROW_FROM and not remat:
                p._v6_packable = True        # the optimizer may emit this weight's packings (captured steps with prepack)
    opt = AdamW6(list(model.parameters()), fmt, lr=lr, tiles=tiles, warps=warps)
    opt.param_groups[0].update(prepack=prepack, pack_warps=pack_warps, mma_warps=mma_warps)
    for layer in plan.narrow:
        _narrow_on_device(layer, plan, opt)
    return model, opt
