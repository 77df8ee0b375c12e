"""LoRA over frozen bases that are kept as they are, re-packed to NVFP4, or loaded as packed NVFP4 checkpoints.

Public surface and behaviour of the reference's src/precision_lora/core.py:
  _FrozenFP4 (core.py:20-63)       mode 'nvfp4': W and W^T are quantised once, each with the sign*H16/4 transform along
                                   its own contraction axis; activations are quantised with the same transform (RNE),
                                   output gradients with the transform and stochastic rounding whose seed is a device
                                   counter that advances after every backward, so graph replays draw fresh noise.
  _LoRAFunction (core.py:66-113)   Y = base(X) + scale * (X A^T) B^T with the low-rank branch accumulated into the base
                                   result in place; dX = base^T(G) + scale * (G B) A; A and B stay FP32 parameters.
  LoRALinear (core.py:116-131), enable_lora (:141-239), lora_parameters (:242-244), prepare_lora (:247-257),
  save_lora / load_lora (:260-303), merge_lora (:306-330).
Mode 'preserve' needs only PyTorch; the NVFP4 modes run on this package's sm_100a kernels.
"""
from __future__ import annotations

import math
import os
import tempfile
from functools import partial
from pathlib import Path

import torch
from torch import nn
from torch.nn import functional as F

from .packed import PackedNVFP4Linear

MODES = ("preserve", "nvfp4", "packed_nvfp4")
_PROTECTED_LEAVES = ("head", "lm_head", "output_layer")
_BASE_DTYPES = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _backend():
    from nvfp4_training._runtime import load_runtime
    backend = load_runtime()[2]
    backend.ensure_verified_modes()
    return backend


class _FrozenFP4(nn.Module):
    """Both orientations of a frozen weight as independent RHT-quantised NVFP4 tensors (no master copy)."""

    def __init__(self, linear, seed):
        super().__init__()
        backend = _backend()
        weight = linear.weight.detach()
        device = weight.device
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.source_dtype = weight.dtype
        self.register_buffer("signs", backend.get_signs(device).clone())
        self.register_buffer("sr_seed", torch.tensor(seed, device=device, dtype=torch.int32))
        if weight.dtype == torch.float16:
            weight = weight.float()
        # the two packings are separate quantisations: scales run along the contraction axis of each product, so the
        # nibbles of one cannot be transposed into the other
        for prefix, source in (("forward", weight), ("backward", weight.t())):
            q = backend.quantize(source, signs=self.signs, rht=True)
            self.register_buffer(prefix + "_data", q.data)
            self.register_buffer(prefix + "_scale", q.scale)
            self.register_buffer(prefix + "_pts", q.pts)
        self.register_buffer("bias", None if linear.bias is None else linear.bias.detach())

    def _weight(self, prefix, dtype):
        from nvfp4_training._backend.quant import Packed
        return Packed(getattr(self, prefix + "_data"), getattr(self, prefix + "_scale"), getattr(self, prefix + "_pts"), dtype)

    def multiply(self, x, backward=False):
        """x @ W^T (+ bias), or for backward g @ W, as one NVFP4 GEMM over freshly quantised x."""
        from nvfp4_training._backend import quant
        if backward:
            # seed = device counter: identical in eager mode and inside a captured graph
            a = quant.quantize(x.contiguous(), signs=self.signs, sr=True, rht=True, seed=0, base=self.sr_seed)
            self.sr_seed.add_(1)
            return quant.matmul(a, self._weight("backward", x.dtype), rows=x.shape[0], cols=self.in_features,
                                output_dtype=x.dtype)
        a = quant.quantize(x, signs=self.signs, rht=True)
        return quant.matmul(a, self._weight("forward", x.dtype), rows=x.shape[0], cols=self.out_features,
                            output_dtype=x.dtype, bias=self.bias)


_NATIVE_BASES = (_FrozenFP4, PackedNVFP4Linear)


class _LoRAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, b, base, scale):
        kind = x.device.type
        compute = torch.get_autocast_dtype(kind) if torch.is_autocast_enabled(kind) else x.dtype
        if isinstance(base, _FrozenFP4) and compute not in (torch.bfloat16, torch.float32):
            raise TypeError("NVFP4 LoRA requires BF16 or FP32 compute; use BF16 autocast")
        if isinstance(base, PackedNVFP4Linear) and compute != torch.bfloat16:
            raise TypeError("Prepacked NVFP4 LoRA requires BF16 compute; use BF16 autocast")
        native = isinstance(base, _NATIVE_BASES)
        # casts are explicit so the adapters stay FP32 and backward does not depend on the autocast state around it
        with torch.autocast(kind, enabled=False):
            rows = x.reshape(-1, x.shape[-1]).to(compute)
            a_c, b_c = a.to(compute), b.to(compute)
            low = F.linear(rows, a_c)
            if native:
                weight = rows.new_empty(0)
                y = base.multiply(rows)
            else:
                weight = base.weight
                y = F.linear(rows, weight.to(compute), None if base.bias is None else base.bias.to(compute))
            y.addmm_(low, b_c.t(), alpha=scale)   # y is private to this call: accumulate in place
        ctx.save_for_backward(rows, low, a_c, b_c, weight)
        ctx.base, ctx.scale, ctx.native = base, scale, native
        ctx.x_shape, ctx.x_dtype, ctx.ab_dtypes = x.shape, x.dtype, (a.dtype, b.dtype)
        return y.reshape(*x.shape[:-1], b.shape[0])

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad):
        rows, low, a_c, b_c, weight = ctx.saved_tensors
        scale = ctx.scale
        with torch.autocast(grad.device.type, enabled=False):
            g = grad.reshape(-1, b_c.shape[0]).to(rows.dtype)
            d_low = g @ b_c
            d_a = torch.mm(d_low.t(), rows)
            d_b = torch.mm(g.t(), low)
            if scale != 1:
                d_a.mul_(scale)
                d_b.mul_(scale)
            d_x = None
            if ctx.needs_input_grad[0]:
                d_x = ctx.base.multiply(g, backward=True) if ctx.native else g @ weight.to(rows.dtype)
                d_x.addmm_(d_low, a_c, alpha=scale)
                d_x = d_x.reshape(ctx.x_shape).to(ctx.x_dtype)
        return d_x, d_a.to(ctx.ab_dtypes[0]), d_b.to(ctx.ab_dtypes[1]), None, None


class LoRALinear(nn.Module):
    """Y = base(X) + (alpha / rank) * X A^T B^T, with B initialised to zero."""

    def __init__(self, linear, rank, alpha, mode, seed):
        super().__init__()
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.rank, self.alpha, self.mode = rank, float(alpha), mode
        device = linear.device if isinstance(linear, PackedNVFP4Linear) else linear.weight.device
        self.base = _FrozenFP4(linear, seed) if mode == "nvfp4" else linear
        self.lora_A = nn.Parameter(torch.empty(rank, self.in_features, device=device, dtype=torch.float32))
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, rank, device=device, dtype=torch.float32))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))

    def forward(self, x):
        if x.shape[-1] != self.in_features:
            raise ValueError("LoRA input feature count does not match the base")
        return _LoRAFunction.apply(x, self.lora_A, self.lora_B, self.base, self.alpha / self.rank)


def _checkpoint_forward(*args, original, **kwargs):
    from torch.utils.checkpoint import checkpoint
    if not torch.is_grad_enabled():
        return original(*args, **kwargs)
    return checkpoint(original, *args, use_reentrant=False, preserve_rng_state=True, **kwargs)


def _overlap(a, b):
    return a == b or a.startswith(b + ".") or b.startswith(a + ".")


def _leaf(name):
    return name.rsplit(".", 1)[-1]


def enable_lora(model, *, mode="preserve", rank=16, alpha=None, target_modules=None, checkpoint_modules=()):
    """Freeze the base, wrap the selected Linear layers and return the model.

    mode 'preserve' keeps the original base Parameters (objects, dtypes, values); 'nvfp4' replaces each selected base
    by two RHT-packed NVFP4 orientations; 'packed_nvfp4' adapts explicit PackedNVFP4Linear modules.
    target_modules: exact paths or last path components (default: every untied Linear except head / lm_head /
    output_layer; a root Linear is allowed).  checkpoint_modules: distinct, non-overlapping parent block paths whose
    forward is recomputed during backward."""
    if (not isinstance(model, nn.Module) or hasattr(model, "nvfp4_optimizer")
            or any(isinstance(m, LoRALinear) for m in model.modules())):
        raise ValueError("Pass an unconverted nn.Module")
    if mode not in MODES:
        raise ValueError("mode must be 'preserve', 'nvfp4' or 'packed_nvfp4'")
    if type(rank) is not int or rank < 1:
        raise ValueError("rank must be a positive integer")
    if alpha is None:
        alpha = rank
    if not math.isfinite(alpha) or alpha <= 0:
        raise ValueError("alpha must be finite and positive")
    if isinstance(target_modules, str) or isinstance(checkpoint_modules, str):
        raise TypeError("Pass a list of module names, not one string")
    wanted = None if target_modules is None else set(target_modules)
    by_path = dict(model.named_modules(remove_duplicate=False))
    blocks = list(checkpoint_modules)
    if (any(not b or b not in by_path for b in blocks)
            or any(_overlap(a, b) for i, a in enumerate(blocks) for b in blocks[:i])):
        raise ValueError("checkpoint_modules must be distinct, non-overlapping existing block paths")
    uses = {}
    for _, t in (*model.named_parameters(remove_duplicate=False), *model.named_buffers(remove_duplicate=False)):
        uses[id(t)] = uses.get(id(t), 0) + 1
    packed_mode = mode == "packed_nvfp4"
    chosen, hit = {}, set()
    for name, module in by_path.items():
        if not isinstance(module, (nn.Linear, PackedNVFP4Linear)):
            continue
        packed = isinstance(module, PackedNVFP4Linear)
        storage = module.packed if packed else module.weight
        if wanted is None:
            take = packed == packed_mode and uses[id(storage)] == 1 and _leaf(name) not in _PROTECTED_LEAVES
        else:
            keys = {name, _leaf(name)} & wanted
            hit |= keys
            take = bool(keys)
        if not take:
            continue
        if packed != packed_mode:
            raise TypeError("packed_nvfp4 targets require PackedNVFP4Linear; floating-point targets use preserve or nvfp4")
        if uses[id(storage)] != 1:
            raise ValueError(f"Target {name!r} shares a weight; leave tied/aliased projections frozen")
        if not packed:
            if type(module) is not nn.Linear:
                raise TypeError(f"Custom Linear at {name!r} requires explicit integration")
            if module.weight.dtype not in _BASE_DTYPES:
                raise TypeError(f"Unsupported base storage at {name!r}: {module.weight.dtype}")
        if mode == "nvfp4" and (module.weight.device.type != "cuda" or module.weight.dtype == torch.float64):
            raise ValueError("NVFP4 targets must be untied FP16/BF16/FP32 CUDA Linear layers")
        chosen[name] = module
    if not chosen or (wanted is not None and hit != wanted):
        raise ValueError(f"No matching Linear, or unmatched targets: {wanted - hit if wanted else wanted}")
    if any(b in chosen for b in blocks):
        raise ValueError("Checkpoint a parent block, not an individual LoRA Linear")
    if mode == "nvfp4":
        _backend()   # fail before anything is frozen or replaced
    for p in model.parameters():
        p.requires_grad_(False)
        p.grad = None
    names = sorted(chosen)
    wrapped = {}
    # each original projection is released as soon as it is replaced, so conversion never holds two full models
    for name in list(chosen):
        module = chosen.pop(name)
        if id(module) not in wrapped:
            wrapped[id(module)] = LoRALinear(module, rank, alpha, mode, len(wrapped) * 100003)
        new = wrapped[id(module)]
        new.train(module.training)
        del module
        if name:
            parent, _, leaf = name.rpartition(".")
            by_path[parent]._modules[leaf] = new
        else:
            model = new
        by_path[name] = new
    for name in blocks:
        block = by_path[name]
        block.forward = partial(_checkpoint_forward, original=block.forward)
    model.lora_config = dict(mode=mode, rank=rank, alpha=float(alpha), targets=names, checkpoint_modules=blocks)
    if packed_mode:
        model.lora_config["packed_layouts"] = {
            n: dict(shape=(by_path[n].in_features, by_path[n].out_features), layout=by_path[n].base.layout,
                    rht_seed=by_path[n].base.rht_seed) for n in names}
    return model


def lora_parameters(model):
    """The trainable adapter parameters, in module order, for any ordinary optimizer."""
    return [p for m in model.modules() if isinstance(m, LoRALinear) for p in (m.lora_A, m.lora_B)]


def prepare_lora(model, *, lr=2e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, **options):
    """(converted model, fused torch AdamW over the FP32 adapters only)."""
    if not all(math.isfinite(v) for v in (lr, eps, weight_decay)) or lr < 0 or eps <= 0 or weight_decay < 0:
        raise ValueError("AdamW requires finite lr >= 0, eps > 0, weight_decay >= 0")
    if len(betas) != 2 or not all(0 <= b < 1 for b in betas):
        raise ValueError("betas must contain two values in [0,1)")
    model = enable_lora(model, **options)
    params = lora_parameters(model)
    optimizer = torch.optim.AdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                  fused=all(p.is_cuda for p in params))
    return model, optimizer


def _adapters(model):
    return {name: m for name, m in model.named_modules() if isinstance(m, LoRALinear)}


def save_lora(path, model, *, optimizer=None, base_id=None):
    """Atomic adapter-only checkpoint (adapters, SR counters, optional optimizer, RNG); bases are never written."""
    rows = {}
    for name, m in _adapters(model).items():
        counter = m.base.sr_seed.cpu() if isinstance(m.base, _NATIVE_BASES) else None
        rows[name] = dict(A=m.lora_A.detach().cpu(), B=m.lora_B.detach().cpu(), sr=counter)
    payload = dict(schema=1, config=model.lora_config, base_id=base_id, adapters=rows,
                   optimizer=None if optimizer is None else optimizer.state_dict(), cpu_rng=torch.get_rng_state(),
                   cuda_rng=torch.cuda.get_rng_state_all() if torch.cuda.is_available() else [])
    path = Path(path)
    with tempfile.NamedTemporaryFile(dir=path.parent, prefix=".lora-", suffix=".tmp", delete=False) as f:
        tmp = Path(f.name)
    try:
        torch.save(payload, tmp)
        os.replace(tmp, path)
    finally:
        tmp.unlink(missing_ok=True)


def _recipe(config):
    return {k: v for k, v in config.items() if k != "checkpoint_modules"}


def load_lora(path, model, *, optimizer=None, base_id=None, restore_rng=True):
    """Restore into the same base and recipe; `base_id`, when given, must equal the saved one."""
    saved = torch.load(path, map_location="cpu", weights_only=True)
    if (saved.get("schema") != 1 or _recipe(saved.get("config", {})) != _recipe(model.lora_config)
            or (base_id is not None and saved.get("base_id") != base_id)):
        raise ValueError("LoRA recipe or base_id mismatch")
    layers, rows = _adapters(model), saved["adapters"]
    if layers.keys() != rows.keys() or any(
            m.lora_A.shape != rows[n]["A"].shape or m.lora_B.shape != rows[n]["B"].shape for n, m in layers.items()):
        raise ValueError("Adapter names or shapes do not match")
    if optimizer is not None and saved["optimizer"] is None:
        raise ValueError("Checkpoint has no optimizer state")
    with torch.no_grad():
        for name, m in layers.items():
            m.lora_A.copy_(rows[name]["A"])
            m.lora_B.copy_(rows[name]["B"])
            if isinstance(m.base, _NATIVE_BASES):
                m.base.sr_seed.copy_(rows[name]["sr"])
    if optimizer is not None:
        optimizer.load_state_dict(saved["optimizer"])
    if restore_rng:
        torch.set_rng_state(saved["cpu_rng"])
        if saved["cuda_rng"]:
            torch.cuda.set_rng_state_all(saved["cuda_rng"])
    return saved.get("base_id")


@torch.no_grad()
def merge_lora(model):
    """Fold the adapters into the original base storage (mode 'preserve' only) and unwrap the layers.

    The sum is rounded to the base dtype, so base values change; keep the adapter checkpoint to resume training."""
    layers = list(_adapters(model).items())
    if any(m.mode != "preserve" for _, m in layers):
        raise ValueError("Merge requires preserve mode and the original floating-point base")
    if len({id(m.base.weight) for _, m in layers}) != len(layers):
        raise ValueError("Cannot merge distinct adapters into a shared base weight")
    for name, m in layers:
        w = m.base.weight
        wide = torch.float64 if w.dtype == torch.float64 else torch.float32
        a = m.lora_A.to(wide)
        for lo in range(0, m.out_features, 256):   # 256 output rows at a time bounds the wide scratch
            rows = slice(lo, lo + 256)
            delta = (m.lora_B[rows].to(wide) @ a) * (m.alpha / m.rank)
            w[rows].copy_((w[rows].to(wide) + delta).to(w.dtype))
        if name:
            parent, _, leaf = name.rpartition(".")
            model.get_submodule(parent)._modules[leaf] = m.base
        else:
            model = m.base
    if hasattr(model, "lora_config"):
        del model.lora_config
    return model
