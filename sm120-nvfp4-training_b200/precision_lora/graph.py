"""One LoRA update (forward, loss, backward, optional clipping, fused AdamW) captured as a CUDA graph.

Interface and guarantees of the reference's LoRAStep (src/precision_lora/graph.py:15-111): constructor arguments, `step`,
`close`, context-manager use and error messages are the same, and capturing never counts as training.  Warm-up and
recording run real updates; `_Rewind` remembers everything such an update touches (adapter weights, optimizer state, the
stochastic-rounding counters of the NVFP4 bases, other module buffers, both RNG states) and puts it back afterwards.  The
SR seed of every NVFP4 base is a device counter incremented inside the graph, so replays draw fresh noise.
"""
from __future__ import annotations

import torch

from .core import _FrozenFP4, lora_parameters
from .packed import PackedNVFP4Linear

_STREAMS = {}


def _capture_stream(device):
    """One side stream per device for every capture: library workspaces are keyed by stream and would pile up otherwise."""
    key = torch.device(device)
    if key not in _STREAMS:
        _STREAMS[key] = torch.cuda.Stream(device=key)
    return _STREAMS[key]


class _Rewind:
    """Values of everything a LoRA update changes, taken at construction; restore() writes them back in place."""

    def __init__(self, optimizer, params, tensors):
        self.optimizer = optimizer
        self.tensors = [(t, t.detach().clone()) for t in (*params, *tensors)]
        self.state = {p: {k: (v.clone() if torch.is_tensor(v) else v) for k, v in optimizer.state.get(p, {}).items()} for p in params}
        self.cuda_rng, self.cpu_rng = torch.cuda.get_rng_state(), torch.get_rng_state()

    @torch.no_grad()
    def restore(self):
        for live, value in self.tensors:
            live.copy_(value)
        for p, before in self.state.items():
            for key, value in self.optimizer.state[p].items():
                if torch.is_tensor(value):      # state created by the warm-up of a fresh optimizer goes back to zero
                    value.copy_(before[key]) if key in before else value.zero_()
        torch.cuda.set_rng_state(self.cuda_rng)
        torch.set_rng_state(self.cpu_rng)


class LoRAStep:
    def __init__(self, model, optimizer, loss_fn, *samples, warmup=3, max_grad_norm=None):
        if any(isinstance(m, PackedNVFP4Linear) for m in model.modules()):
            raise ValueError("packed_nvfp4 currently uses eager training; CUDA graph replay has not been validated")
        if type(warmup) is not int or warmup < 2:
            raise ValueError("Use at least two warmup steps")
        params = lora_parameters(model)
        if not params or any(not p.is_cuda or p.device != params[0].device for p in params):
            raise ValueError("CUDA LoRA model required")
        device = params[0].device
        groups = optimizer.param_groups if isinstance(optimizer, torch.optim.AdamW) else None
        if groups is None or not all(g.get("fused") for g in groups):
            raise ValueError("LoRA capture requires fused torch.optim.AdamW")
        if {id(p) for p in params} != {id(p) for g in groups for p in g["params"]}:
            raise ValueError("Optimizer must contain exactly the LoRA parameters")
        if any(not torch.is_tensor(t) or t.device != device for t in samples):
            raise ValueError("Pass fixed-shape CUDA tensor inputs")
        self.model, self.optimizer, self.params = model, optimizer, params
        self.loss_fn, self.max_grad_norm = loss_fn, max_grad_norm
        self.inputs = [t.detach().clone() for t in samples]
        self.closed, self.original_training = False, model.training
        self.capture_flags = [g.get("capturable", False) for g in groups]
        for g in groups:
            g["capturable"] = True          # the fused optimizer then keeps its step counters on the device
        bases = [m for m in model.modules() if isinstance(m, _FrozenFP4)]
        self.seed_buffers = [m.sr_seed for m in bases]
        owned_by_bases = {id(b) for m in bases for b in m.buffers()}
        self.other_buffers = [b for b in model.buffers() if id(b) not in owned_by_bases]
        rewind = _Rewind(optimizer, params, (*self.seed_buffers, *self.other_buffers))
        side, main = _capture_stream(device), torch.cuda.current_stream()
        side.wait_stream(main)
        try:
            with torch.cuda.stream(side):
                for _ in range(warmup):
                    self._update()
            main.wait_stream(side)
            torch.cuda.synchronize()
            rewind.restore()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._update()
            rewind.restore()
            optimizer.zero_grad(set_to_none=False)
        except BaseException:
            torch.cuda.synchronize()
            rewind.restore()
            self._restore_flags()
            raise

    def _update(self):
        self.optimizer.zero_grad(set_to_none=False)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = self.loss_fn(self.model, *self.inputs)
        loss.backward()
        if self.max_grad_norm is not None:
            torch.nn.utils.clip_grad_norm_(self.params, self.max_grad_norm)
        self.optimizer.step()
        self.loss = loss.detach()

    def _restore_flags(self):
        for group, flag in zip(self.optimizer.param_groups, self.capture_flags):
            group["capturable"] = flag

    def step(self, *batch):
        if self.closed:
            raise RuntimeError("LoRA graph is closed")
        if self.model.training != self.original_training:
            raise RuntimeError("Do not change train/eval mode during graph replay")
        matches = len(batch) == len(self.inputs) and all(
            given.shape == held.shape and given.dtype == held.dtype and given.device == held.device for given, held in zip(batch, self.inputs))
        if not matches:
            raise ValueError("Graph inputs must match the captured shape, dtype and device")
        for held, given in zip(self.inputs, batch):
            held.copy_(given)
        self.graph.replay()
        return self.loss.detach()

    def close(self):
        if self.closed:
            return
        torch.cuda.synchronize()
        self.closed = True
        self.graph.reset()
        self.optimizer.zero_grad(set_to_none=True)
        self._restore_flags()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def capture_lora_step(model, optimizer, loss_fn, *samples, **options):
    return LoRAStep(model, optimizer, loss_fn, *samples, **options)
