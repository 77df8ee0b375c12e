"""B200 (sm_100a) implementation of the `nvfp4_training` interface.

Same public names, arguments, defaults and exceptions as the reference package (src/nvfp4_training/__init__.py:12-193);
host code is Python / PyTorch, every NVFP4 kernel is hand-written CUDA behind the C ABI of include/nvfp4_b200.h.
"""
from .profiles import list_profiles, profile_config
from ._runtime import load_runtime

__all__ = ["list_profiles", "prepare_training", "enable_nvfp4", "train_step", "capture_step", "save_checkpoint", "load_checkpoint",
           "check_finite", "enable_lora", "prepare_lora", "lora_parameters", "save_lora", "load_lora", "merge_lora",
           "capture_lora_step", "PackedNVFP4Linear", "pack_frozen_layers", "save_frozen_cache", "load_frozen_cache", "capture_frozen",
           "enable_data_parallel"]

_LORA = {"enable_lora", "prepare_lora", "lora_parameters", "save_lora", "load_lora", "merge_lora", "PackedNVFP4Linear", "capture_lora_step"}


def __getattr__(name):
    # LoRA entry points live in precision_lora (as in the reference); imported on first use
    if name in _LORA:
        from . import lora
        return getattr(lora, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def pack_frozen_layers(model, *, include, keep=()):
    from .frozen import pack_frozen_layers as convert
    return convert(model, include=include, keep=keep)


def save_frozen_cache(path, model, *, model_fingerprint):
    from .frozen import save_frozen_cache as save
    return save(path, model, model_fingerprint=model_fingerprint)


def load_frozen_cache(path, model, *, expected_fingerprint, device='cuda'):
    from .frozen import load_frozen_cache as load
    return load(path, model, expected_fingerprint=expected_fingerprint, device=device)


def capture_frozen(model, compute, *inputs, backward=True, warmup=2):
    from .frozen import capture_frozen as capture
    return capture(model, compute, *inputs, backward=backward, warmup=warmup)


def enable_data_parallel(model, process_group=None, *, bucket_mb=25.0, depth=2, peer_timeout=None):
    """Data-parallel replicas: NCCL all-reduce of the gradients, overlapped with backward.  Weight gradients of converted
    layers are reduced in place, one collective each; small dense gradients share FP32 buckets of bucket_mb megabytes.
    Ranks must agree on the converted layers (checked here, on the host); peer_timeout (seconds) adds a host-side liveness
    check before every eager step.  nvfp4_training.distributed.verify_replicas compares a digest of all state."""
    from .distributed import enable_data_parallel as enable
    return enable(model, process_group, bucket_mb=bucket_mb, depth=depth, peer_timeout=peer_timeout)


def prepare_training(model, *, profile="balanced", precision="fp4", remat=False, lr=1e-4, betas=(0.9, 0.999), eps=1e-8,
                     weight_decay=0.01):
    """Convert a fresh FP32 model in place and return (model, matching AdamW)."""
    from ._convert import prepare
    return prepare(model, profile=profile, precision=precision, remat=remat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)


def enable_nvfp4(model, *, profile="balanced", **options):
    """Return the converted model; its optimizer is model.nvfp4_optimizer."""
    return prepare_training(model, precision="fp4", profile=profile, **options)[0]


def _loss(model, fn, *batch):
    import torch
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = fn(model, *batch)
    if not isinstance(loss, torch.Tensor) or loss.ndim != 0 or not loss.requires_grad:
        raise ValueError("loss_fn(model, *batch) must return a scalar loss with gradients")
    return loss


def train_step(model, loss_fn, *batch):
    """One eager step on CUDA inputs; dimensions can vary between steps."""
    opt = model.nvfp4_optimizer
    opt.zero_grad(set_to_none=True)
    loss = _loss(model, loss_fn, *batch)
    opt.backward_step(loss)
    return loss.detach()


def capture_step(model, loss_fn, x, y, *, steps):
    """Capture fixed-shape forward, loss, backward and AdamW.  Use as a context manager."""
    if type(steps) is not int or steps < 1:
        raise ValueError("steps must be a positive integer")
    opt = model.nvfp4_optimizer
    step_cls = load_runtime()[1]
    untrained = not any(state.get("step", 0) for state in opt.state.values())
    return step_cls(model, opt, lambda a, b: _loss(model, loss_fn, a, b), x, y, steps, stream_updates=True, from_start=untrained)


def save_checkpoint(path, model):
    """Atomically save model, optimizer, CPU/CUDA RNG and the NVFP4 SR counter."""
    from ._checkpoint import save
    save(path, model)


def load_checkpoint(path, model):
    """Restore into a freshly prepared matching model.  Returns the restored optimizer step."""
    from ._checkpoint import load
    return load(path, model)


def check_finite(model):
    """Explicit diagnostic over all parameters, buffers and floating optimizer states (and the kernels' status word)."""
    from ._checkpoint import check_finite as check
    check(model)
