"""One LoRA update (forward, loss, backward, optional clipping, fused AdamW) captured as a CUDA graph.

Follows the reference's LoRAStep (src/precision_lora/graph.py:15-111): warm-up and capture run real updates, after
which parameters, optimizer state, stochastic-rounding counters, other buffers and both RNG states are put back, so
capturing never counts as training.  The SR seed of every NVFP4 base is a device counter incremented inside the graph.
"""
from __future__ import annotations

from functools import lru_cache

import torch

from .core import _FrozenFP4, lora_parameters
from .packed import PackedNVFP4Linear


@lru_cache(maxsize=None)
def _capture_stream(device):
    # one side stream per device for every capture: library workspaces are keyed by stream and would pile up otherwise
    return torch.cuda.Stream(device=device)


def _snapshot(tensors):
    return [t.detach().clone() for t in tensors]


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
        if not isinstance(optimizer, torch.optim.AdamW) or any(not g.get("fused") for g in optimizer.param_groups):
            raise ValueError("LoRA capture requires fused torch.optim.AdamW")
        if {id(p) for p in params} != {id(p) for g in optimizer.param_groups for p in g["params"]}:
            raise ValueError("Optimizer must contain exactly the LoRA parameters")
        if any(not torch.is_tensor(t) or t.device != device for t in samples):
            raise ValueError("Pass fixed-shape CUDA tensor inputs")
        self.model, self.optimizer, self.params = model, optimizer, params
        self.capture_flags = [g.get("capturable", False) for g in optimizer.param_groups]
        for group in optimizer.param_groups:
            group["capturable"] = True
        self.inputs = [t.detach().clone() for t in samples]
        self.closed = False
        self.original_training = model.training
        bases = [m for m in model.modules() if isinstance(m, _FrozenFP4)]
        self.seed_buffers = [m.sr_seed for m in bases]
        frozen_ids = {id(b) for m in bases for b in m.buffers()}
        self.other_buffers = [b for b in model.buffers() if id(b) not in frozen_ids]
        kept = dict(params=_snapshot(params), seeds=_snapshot(self.seed_buffers), buffers=_snapshot(self.other_buffers),
                    cuda_rng=torch.cuda.get_rng_state(), cpu_rng=torch.get_rng_state(),
                    state={p: {k: v.clone() if torch.is_tensor(v) else v for k, v in optimizer.state.get(p, {}).items()}
                           for p in params})   # a started optimizer is preserved too

        def update():
            optimizer.zero_grad(set_to_none=False)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = loss_fn(model, *self.inputs)
            loss.backward()
            if max_grad_norm is not None:
                torch.nn.utils.clip_grad_norm_(params, max_grad_norm)
            optimizer.step()
            self.loss = loss.detach()

        @torch.no_grad()
        def rewind():
            for group, values in ((params, kept["params"]), (self.seed_buffers, kept["seeds"]),
                                  (self.other_buffers, kept["buffers"])):
                for t, value in zip(group, values):
                    t.copy_(value)
            for p, before in kept["state"].items():
                for key, value in optimizer.state[p].items():
                    if torch.is_tensor(value):
                        if key in before:
                            value.copy_(before[key])
                        else:
                            value.zero_()
            torch.cuda.set_rng_state(kept["cuda_rng"])
            torch.set_rng_state(kept["cpu_rng"])

        side = _capture_stream(device)
        side.wait_stream(torch.cuda.current_stream())
        try:
            with torch.cuda.stream(side):
                for _ in range(warmup):
                    update()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            rewind()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                update()
            rewind()
            optimizer.zero_grad(set_to_none=False)
        except BaseException:
            torch.cuda.synchronize()
            rewind()
            self._restore_flags()
            raise

    def _restore_flags(self):
        for group, flag in zip(self.optimizer.param_groups, self.capture_flags):
            group["capturable"] = flag

    def step(self, *batch):
        if self.closed:
            raise RuntimeError("LoRA graph is closed")
        if self.model.training != self.original_training:
            raise RuntimeError("Do not change train/eval mode during graph replay")
        if len(batch) != len(self.inputs) or any(
                a.shape != b.shape or a.dtype != b.dtype or a.device != b.device for a, b in zip(batch, self.inputs)):
            raise ValueError("Graph inputs must match the captured shape, dtype and device")
        for dst, src in zip(self.inputs, batch):
            dst.copy_(src)
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
