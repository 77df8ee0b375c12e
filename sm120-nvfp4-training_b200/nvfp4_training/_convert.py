"""Conversion of a fresh FP32 model into an NVFP4-trained one: argument and model validation, then engine.configure.

The checks, their order, exception types and messages are those of the reference's prepare_training
(src/nvfp4_training/__init__.py:34-93), which callers and tests rely on; they are written here as a list of rules that is
walked once, so that every rule states its condition, its exception and its message in one place.
"""
import math

import torch
from torch import nn

from ._runtime import load_runtime
from .profiles import profile_config


def _argument_rules(precision, remat, lr, betas, eps, weight_decay):
    finite = all(isinstance(v, (int, float)) and math.isfinite(v) for v in (lr, eps, weight_decay))
    return (
        (precision in ("fp4", "bf16") and type(remat) is bool, ValueError, "precision must be 'fp4' or 'bf16', and remat must be a bool"),
        (not (remat and precision == "bf16"), ValueError, "remat applies to NVFP4 transpose encoding; use remat=False for BF16"),
        (isinstance(betas, (tuple, list)) and len(betas) == 2 and all(0 <= b < 1 for b in betas), ValueError,
         "betas must contain two numbers in [0, 1)"),
        (finite and lr >= 0 and eps > 0 and weight_decay >= 0, ValueError, "AdamW requires finite lr >= 0, eps > 0 and weight_decay >= 0"),
    )


def _model_rules(model):
    """Evaluated lazily, one after the other: later rules may assume the earlier ones hold."""
    yield (lambda: isinstance(model, nn.Module) and not hasattr(model, "nvfp4_optimizer"), ValueError,
           "Pass a fresh, unconverted torch.nn.Module")
    params = list(model.parameters()) if isinstance(model, nn.Module) else []
    yield (lambda: bool(params) and any(type(m) is nn.Linear for m in model.modules()), ValueError,
           "The model must contain a standard nn.Linear")
    yield (lambda: not any(isinstance(m, nn.Linear) and type(m) is not nn.Linear for m in model.modules()), TypeError,
           "Custom Linear subclasses and previously converted submodules require explicit integration")

    def placed():
        device = params[0].device
        return device.type in ("cpu", "cuda") and all(
            p.device == device and p.dtype == torch.float32 and p.is_contiguous() and p.requires_grad and p.numel() for p in params)
    yield (placed, ValueError, "Expected trainable, nonempty, contiguous FP32 parameters on one CPU or CUDA device")
    yield (lambda: len({p.untyped_storage().data_ptr() for p in params}) == len(params), ValueError,
           "Tie weights using the same Parameter object, not distinct views of one storage")


def _enforce(rules):
    for condition, error, message in rules:
        if not (condition() if callable(condition) else condition):
            raise error(message)


def prepare(model, *, profile, precision, remat, lr, betas, eps, weight_decay):
    cfg = profile_config(profile)
    _enforce(_argument_rules(precision, remat, lr, betas, eps, weight_decay))
    _enforce(_model_rules(model))
    engine, _, counters, linear_cls = load_runtime()
    fp4 = precision == "fp4"
    if fp4:
        counters.ensure_verified_modes()
    on_cpu = next(model.parameters()).device.type == "cpu"
    direct = on_cpu and cfg.direct_cpu          # narrow masters are made on the host and only they travel to the GPU
    if on_cpu and not direct:
        model = model.cuda()
    model, opt = engine.configure(model, precision, cfg.storage, lr=lr, tiles=cfg.tiles, warps=cfg.warps, direct=direct, remat=remat,
                                  act_pair=fp4, fast_scale=fp4, mma_k=128 if fp4 and cfg.short_mma_warps else 0,
                                  mma_warps=cfg.short_mma_warps or 8)
    if fp4:
        for module in model.modules():
            if isinstance(module, engine.Linear6):
                module.__class__ = linear_cls
    for target in (opt.defaults, opt.param_groups[0]):
        target.update(betas=tuple(betas), eps=eps, weight_decay=weight_decay)
    model.nvfp4_optimizer, model.nvfp4_profile, model.nvfp4_precision, model.nvfp4_remat = opt, profile, precision, remat
    return model, opt
