"""A whole training step (forward, loss, backward, optimizer updates) recorded once as a CUDA graph and replayed.

Interface and guarantees are those of the reference's StaticStep (src/nvfp4_training/_backend/step6.py:9-174): same
constructor arguments, `step(x, y)`, `close()`, context-manager use, `sr_calls`, and the same error messages when the
model, the optimizer or the batch layout changed under a capture.  What a replay needs to differ from the previous one
(bias corrections, step number, the base of the stochastic-rounding seeds) travels through a four-float control tensor
that the kernels read on the device, so one recording serves `steps` consecutive updates.

This backend adds three things the recording has to arrange: the main line is recorded on a high-priority stream and
the optimizer updates on a second one that forks at every finished gradient (optimizer.capture_streaming_backward);
pools that hold capture-private memory (the activation-packing memo, amax slots) are emptied at both ends of the
recording; and with `prepack` the weights' NVFP4 packings live in buffers that the update kernels keep current.
"""
from __future__ import annotations

import math
from types import SimpleNamespace

import torch

from .. import _native
from . import quant as rng
from .linear import Linear6, decoded
from .optimizer import AdamW

_FROZEN_SETTINGS = ('lr', 'betas', 'eps', 'weight_decay', 'compact', 'cache_scale', 'format', 'tiles', 'warps', 'prepack',
                    'pack_warps', 'state_block', 'mma_warps')


class StaticStep:
    """Owns a captured training step for a bounded number of optimizer updates.  Keep model structure, optimizer
    group and batch layout fixed; close() before eager training or checkpointing."""

    def __init__(self, model, optimizer, compute, x, y, steps, *, stream_updates=False, from_start=False):
        if not isinstance(optimizer, AdamW) or len(optimizer.param_groups) != 1 or steps < 1:
            raise ValueError("One warmed v5 AdamW group and a positive replay count required")
        self.model, self.opt, self.steps, self.index = model, optimizer, steps, 0
        self.group = optimizer.param_groups[0]
        self.params = tuple(self.group['params'])
        self.config = self._settings()
        self.device = x.device
        self._check_ownership(model, x, y)
        self.start = self._common_step(from_start)
        self.training = model.training
        self.stream = torch.cuda.current_stream(self.device)
        self.closed = False
        self.x, self.y = x.detach().clone(), y.detach().clone()
        self.ctrl = torch.empty(4, device=self.device, dtype=torch.float32)
        owners = [p for p in self.params if getattr(p, '_v4_request_scale', False)]
        if owners and not any(isinstance(m, Linear6) for m in model.modules()):
            raise ValueError("Use the NVFP4 converter for replay-safe SR")
        if getattr(optimizer, '_graph_owner', None) is not None:
            raise RuntimeError("Optimizer is already captured")
        self.scales = self._persistent_scales(owners, from_start)
        self.packs = self._persistent_packings(owners)
        optimizer.zero_grad(set_to_none=True)
        overlapped = stream_updates and optimizer.overlap_updates
        self.graph = torch.cuda.CUDAGraph()
        self._record(compute, owners, stream_updates, overlapped, from_start)
        if owners and self.sr_calls == 0:
            raise RuntimeError("No dynamic SR in FP4 backward")
        self._plan_replays()
        optimizer._graph_owner = self
        self.versions = tuple(p._version for p in self.params)
        self.pointers = tuple(p.data_ptr() for p in self.params)

    # ---- what must hold before anything is recorded -------------------------------------------------------------------
    def _settings(self):
        return tuple(self.group.get(k) for k in _FROZEN_SETTINGS)

    def _check_ownership(self, model, x, y):
        one_device = self.device.type == 'cuda' and y.device == self.device and not (x.requires_grad or y.requires_grad)
        if not one_device or any(p.device != self.device or not p.requires_grad for p in self.params):
            raise ValueError("StaticStep requires one device, trainable parameters and data-only inputs")
        if {id(p) for p in model.parameters() if p.requires_grad} != {id(p) for p in self.params}:
            raise ValueError("Optimizer must own every trainable parameter of this model")

    def _common_step(self, from_start):
        state = self.opt.state
        if from_start:
            if any(state.get(p, {}).get("step", 0) for p in self.params):
                raise ValueError("from_start requires a new optimizer")
            for p in self.params:
                self.opt._state_for(p, self.group)
        counts = {state.get(p, {}).get('step', 0) for p in self.params}
        if len(counts) != 1 or (not from_start and min(counts) < 1):
            raise ValueError("Warm up all parameters together before capture")
        return counts.pop()

    def _persistent_scales(self, owners, from_start):
        """Every converted weight's tensor scale as a tensor that outlives the recording: the update kernels write the next
        scale into it, the next replay's forward reads it."""
        scales = {}
        if not self.group['cache_scale']:
            return scales
        here = self.stream.cuda_stream
        for p in owners:
            cached = getattr(p, '_v4_scale', None)
            if cached is not None and cached[:3] == (p._version, p.data_ptr(), here):
                scales[p] = cached[3]
            elif from_start:
                with torch.no_grad():
                    image = decoded(p) if p.dtype == torch.float8_e4m3fn else p.detach()
                    scales[p] = rng.weight_scale(image).clone()
            else:
                raise ValueError("Warm up on this stream after the last parameter edit")
        return scales

    def _persistent_packings(self, owners):
        """prepack: both NVFP4 orientations of each weight in buffers that the optimizer's kernels rewrite after every
        update (filled here once from the present weights), so that the recorded forward holds no weight quantiser."""
        holders = []
        if not (self.group.get('prepack', False) and self.group['cache_scale']):
            return holders
        with torch.no_grad():
            for p in owners:
                fits = getattr(p, '_v6_packable', False) and p in self.scales and p.ndim == 2 and p.is_contiguous()
                if fits and p.dtype != torch.float8_e4m3fn:
                    d, s, _, dt, st = rng.pair(p.detach(), self.scales[p])
                    p._v6_pack = dict(buffers=(d, s, dt, st), version=p._version, scale=self.scales[p])
                    holders.append(p)
        return holders

    # ---- the recording ------------------------------------------------------------------------------------------------
    def _record(self, compute, owners, stream_updates, overlapped, from_start):
        opt = self.opt
        # captured kernel nodes inherit the stream's priority: the main line is placed before the overlapped updates
        side = torch.cuda.Stream(device=self.device, priority=-1 if overlapped else 0)
        side.wait_stream(self.stream)
        with torch.cuda.stream(side):
            if from_start:
                # libraries create handles and workspaces on first use and may not allocate while a capture is open
                torch.cuda.current_blas_handle()
                probe = torch.ones((16, 16), device=self.device, dtype=torch.bfloat16, requires_grad=True)
                (probe @ probe).sum().backward()
                del probe
            _native.scratch(self.device)         # per-stream scratch and the status word exist before the capture
            _native.status_word(self.device)
        if overlapped:
            opt.update_stream(self.device).synchronize()
        side.synchronize()
        clock = SimpleNamespace(sr_calls=0, seed=self.ctrl[2:3].view(torch.int32))
        try:
            for p in owners:
                p._v5_clock = clock
            for p, scale in self.scales.items():
                p._v5_graph_scale = scale
            opt._graph_control = self.ctrl
            rng.remember_in_capture(True)
            before = _native.CALLS
            with torch.cuda.graph(self.graph, stream=side):
                self.loss = compute(self.x, self.y)
                (opt.capture_streaming_backward if stream_updates else opt.backward_step)(self.loss)
            self.library_calls = _native.CALLS - before    # C-ABI calls in the graph: one or two kernels each
            self.loss = self.loss.detach()
            if any(opt.state[p]['step'] != self.start + 1 for p in self.params):
                raise RuntimeError("Every owned parameter must participate in the captured step")
        finally:
            rng.remember_in_capture(False)
            for p in owners:
                del p._v5_clock
            for p in self.scales:
                del p._v5_graph_scale
            del opt._graph_control
            for p in self.params:
                opt.state[p]['step'] = self.start     # recording is not training: the counters move with the replays
        self.sr_calls = clock.sr_calls

    def _plan_replays(self):
        """Control rows, one per replay: 1 / (1 - b1^t), 1 / sqrt(1 - b2^t), bits of the SR seed base, bits of t."""
        b1, b2 = self.group['betas']
        t = torch.arange(self.start + 1, self.start + self.steps + 1, dtype=torch.float64)
        plan = torch.empty((self.steps, 4), dtype=torch.float32)
        plan[:, 0] = torch.tensor([1 / (1 - b1 ** int(k)) for k in t])
        plan[:, 1] = torch.tensor([1 / math.sqrt(1 - b2 ** int(k)) for k in t])
        self.seed0 = rng._SEED
        bases = (self.seed0 + torch.arange(self.steps, dtype=torch.int64) * self.sr_calls).to(torch.int32)
        plan[:, 2] = bases.view(torch.float32)
        plan[:, 3] = t.to(torch.int32).view(torch.float32)
        self.schedule = plan.to(self.device)
        self.seed_end = (self.seed0 + self.steps * self.sr_calls) & 0xffffffff
        rng._SEED = self.seed_end

    # ---- replay ---------------------------------------------------------------------------------------------------------
    def step(self, x, y):
        groups = self.opt.param_groups
        if self.model.training != self.training or len(groups) != 1 or groups[0] is not self.group:
            raise RuntimeError("Captured training mode and parameter group must stay fixed")
        if self.closed or self.index >= self.steps:
            raise RuntimeError("Capture closed or schedule exhausted")
        if torch.cuda.current_stream(self.device) != self.stream or self._settings() != self.config:
            raise RuntimeError("Captured optimizer settings and stream must stay fixed")
        if tuple(p._version for p in self.params) != self.versions or tuple(p.data_ptr() for p in self.params) != self.pointers:
            raise RuntimeError("Parameter edited outside captured step")
        for given, held in ((x, self.x), (y, self.y)):
            if given.device != held.device or given.dtype != held.dtype or given.shape != held.shape or given.requires_grad:
                raise ValueError("Batch device, shape and dtype must match capture")
            held.copy_(given)
        self.ctrl.copy_(self.schedule[self.index])
        self.graph.replay()
        torch.autograd.graph.increment_version(self.params)
        self.versions = tuple(p._version for p in self.params)
        self.index += 1
        return self.loss.detach()

    def close(self):
        if self.closed:
            return
        here = self.stream.cuda_stream
        for p, version, pointer in zip(self.params, self.versions, self.pointers):
            self.opt.state[p]['step'] = self.start + self.index
            if p in self.scales and p._version == version and p.data_ptr() == pointer:
                p._v4_scale = (p._version, p.data_ptr(), here, self.scales[p])      # eager training carries on from here
            elif hasattr(p, '_v4_scale'):
                del p._v4_scale
        for p in self.packs:
            if hasattr(p, '_v6_pack'):
                del p._v6_pack
        if self.sr_calls and rng._SEED == self.seed_end:
            rng._SEED = (self.seed0 + self.index * self.sr_calls) & 0xffffffff       # hand back the unused seeds
        del self.opt._graph_owner
        self.closed = True
        self.opt.zero_grad(set_to_none=True)
        self.graph.reset()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()
