"""Training checkpoints: one file holding model, optimizer, both RNG states and the stochastic-rounding counter.

Layout and checks follow the reference (src/nvfp4_training/__init__.py:127-168): {"schema": 1, "recipe": (profile, precision,
remat), "model", "optimizer", "sr", "cpu_rng", "cuda_rng"}; a checkpoint only loads into a freshly prepared model of the same
recipe and structure, and the first update after loading is byte-identical to the update the saving process would have made.
"""
import os
import tempfile
from pathlib import Path

import torch

from ._runtime import load_runtime

SCHEMA = 1


def recipe_of(model):
    return (model.nvfp4_profile, model.nvfp4_precision, model.nvfp4_remat)


def save(path, model):
    path = Path(path)
    payload = {"schema": SCHEMA, "recipe": recipe_of(model), "model": model.state_dict(),
               "optimizer": model.nvfp4_optimizer.state_dict(),          # refuses while a captured step is open
               "sr": int(load_runtime()[2]._SEED), "cpu_rng": torch.get_rng_state(),
               "cuda_rng": torch.cuda.get_rng_state(next(model.parameters()).device)}
    # written beside the target and renamed over it: a reader never sees half a file
    handle, scratch = tempfile.mkstemp(dir=path.parent, prefix=".nvfp4-", suffix=".tmp")
    os.close(handle)
    try:
        torch.save(payload, scratch)
        os.replace(scratch, path)
    finally:
        Path(scratch).unlink(missing_ok=True)


def _same_layout(name, have, saved):
    if have.dtype != saved.dtype:
        return False
    # FP8 masters once stored one scalar unit per weight; such files still load (the scalar is spread over the blocks)
    legacy_unit = name.rsplit(".", 1)[-1] == "_v6_unit_buffer" and saved.ndim == 0 and have.ndim == 1
    return have.shape == saved.shape or legacy_unit


def load(path, model):
    opt = model.nvfp4_optimizer
    opt._require_eager()
    saved = torch.load(path, map_location="cpu", weights_only=True)
    if saved.get("schema") != SCHEMA or tuple(saved.get("recipe", ())) != recipe_of(model):
        raise ValueError("Checkpoint profile, precision or remat does not match the prepared model")
    current, stored = model.state_dict(), saved["model"]
    if current.keys() != stored.keys() or not all(_same_layout(k, v, stored[k]) for k, v in current.items()):
        raise ValueError("Checkpoint model structure, dtype or shape mismatch")
    groups = saved["optimizer"]["param_groups"]
    if len(groups) != 1 or len(groups[0]["params"]) != len(opt.param_groups[0]["params"]):
        raise ValueError("Checkpoint optimizer parameter group mismatch")
    model.load_state_dict(stored)
    opt.load_state_dict(saved["optimizer"])
    load_runtime()[2].reset_stats(saved["sr"])
    torch.set_rng_state(saved["cpu_rng"])
    torch.cuda.set_rng_state(saved["cuda_rng"], next(model.parameters()).device)
    return max((state.get("step", 0) for state in opt.state.values()), default=0)


def check_finite(model):
    """Raises FloatingPointError naming every parameter, buffer and floating optimizer state that holds a NaN or an
    infinity (for FP8 masters: a NaN code), then reports a kernel whose bounded device-side wait expired."""
    from . import _native
    opt = model.nvfp4_optimizer
    names, flags = [], []

    def inspect(name, tensor):
        if torch.is_tensor(tensor) and tensor.is_floating_point():
            data = tensor.detach()
            healthy = ((data.view(torch.uint8) & 127) != 127).all() if data.dtype == torch.float8_e4m3fn else torch.isfinite(data).all()
            names.append(name)
            flags.append(healthy)
    for name, p in model.named_parameters():
        inspect(name, p)
        for key, value in opt.state.get(p, {}).items():
            inspect(f"{name}.{key}", value)
    for name, buffer in model.named_buffers():
        inspect(name, buffer)
    verdicts = torch.stack(flags).tolist()      # one synchronisation for the whole model
    broken = [name for name, ok in zip(names, verdicts) if not ok]
    if broken:
        raise FloatingPointError("Nonfinite training tensors: " + ", ".join(broken))
    _native.check_status()
