"""AdamW with compressed state, one fused kernel per parameter.

State layout, hyper-parameter arithmetic, random-bit keys and the backward-time update protocol follow the reference
(src/nvfp4_training/_backend/optimizer_v5.py:66-240 and engine6.py:13-207) so that optimizer checkpoints are
interchangeable; the kernels are nvfp4_adamw_step / nvfp4_adamw_plain of the C-ABI library.
"""
from __future__ import annotations

import math

import torch

from .. import _native as nat

# storage format -> (master encoding, variance bits, momentum bits)
FORMATS = {'tile32': (32, 16, 8), 'fp32_v8': (32, 8, 8), 'split24_v16': (24, 16, 8), 'split24_v8': (24, 8, 8), 'sr16_v8': (16, 8, 8),
           'split24_m4': (24, 8, 4), 'sr16_m4': (16, 8, 4), 'sr16_m4v4': (16, 4, 4), 'float8_v8': (8, 8, 8),
           'half16_v16': (17, 16, 8), 'half16_v8': (17, 8, 8), 'half16_m8v4': (17, 4, 8), 'half16_m4v4': (17, 4, 4),
           'half16_m4v4_sqrt': (17, 4, 4), 'float8_m4v4_sqrt': (8, 4, 4), 'half16_v8b64': (17, 8, 8), 'half16_v8b128': (17, 8, 8),
           'half16_v8b256': (17, 8, 8)}
BLOCK = 512


def state_block(fmt: str) -> int:
    return int(fmt.split('v8b')[1]) if 'v8b' in fmt else BLOCK


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


class AdamW(torch.optim.Optimizer):
    """FP32 updates; tensors of at least 4096 elements keep block-scaled INT8 / FP16 moments."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, *, compact=True, cache_scale=True):
        if not (lr >= 0 and eps > 0 and weight_decay >= 0 and all(0 <= b < 1 for b in betas)):
            raise ValueError("Invalid AdamW hyperparameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, compact=compact, cache_scale=cache_scale))
        self.reducer = None  # data-parallel gradient reducer, attached by nvfp4_training.distributed

    # ---- bookkeeping shared by eager and captured steps -------------------------------------------------
    def _require_eager(self):
        if getattr(self, "_graph_owner", None) is not None:
            raise RuntimeError("Close StaticStep before eager updates or checkpointing")

    def zero_grad(self, set_to_none=True):
        self._require_eager()
        return super().zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        self._require_eager()
        return super().state_dict()

    def load_state_dict(self, state_dict):
        # Optimizer.load_state_dict casts floating states to the parameter dtype; encoded tensors must keep theirs.
        self._require_eager()
        super().load_state_dict(state_dict)
        for saved, group in zip(state_dict['param_groups'], self.param_groups):
            for key, p in zip(saved['params'], group['params']):
                original = state_dict['state'].get(key)
                if original:
                    self.state[p] = {k: v.to(device=p.device, copy=True) if torch.is_tensor(v) else v for k, v in original.items()}
                if hasattr(p, '_v4_scale'):
                    del p._v4_scale

    def _hyper(self, g, t):
        b1, b2 = g['betas']
        return dict(lr=g['lr'], decay=1 - g['lr'] * g['weight_decay'], b1=b1, b2=b2, c1=1 / (1 - b1 ** t),
                    c2=1 / math.sqrt(1 - b2 ** t), eps=g['eps'])

    def _state_for(self, p, g):
        n = p.numel()
        compact = g["compact"] and n >= 4096
        s = self.state[p]
        if not s:
            s['step'] = 0
            s['m'] = torch.zeros_like(p, dtype=torch.int8 if compact else torch.float32)
            s['v'] = torch.zeros_like(p, dtype=torch.float16 if compact else torch.float32)
            if compact:
                for name in ('ms', 'vs'):
                    s[name] = torch.ones(cdiv(n, BLOCK), device=p.device, dtype=torch.float32)
        return s

    def _grad_mul(self):
        return 1.0 if self.reducer is None else self.reducer.grad_scale

    # ---- updates overlapped with the rest of backward (captured steps) ------------------------------------
    #: Under capture, parameter updates are recorded on a second stream that forks after the parameter's gradient is
    #: complete and joins at the end of backward.  The AdamW kernel is bound by integer / FP32 instruction issue and
    #: the GEMMs, attention and copies around it are not, so the graph may run them on the same SMs at once.  Results
    #: do not change: same kernels on the same values, only their placement in the graph.
    overlap_updates = True

    def update_stream(self, device):
        """The stream captured updates are recorded on (created on first use, with its amax scratch)."""
        streams = self.__dict__.setdefault("_update_streams", {})
        key = torch.device(device).index
        if key not in streams:
            streams[key] = torch.cuda.Stream(device=device)
            with torch.cuda.stream(streams[key]):
                nat.scratch(torch.device(device))
        return streams[key]

    def _overlapping(self):
        return self.overlap_updates and torch.cuda.is_current_stream_capturing()

    def _update_overlapped(self, p, group, pack, work=None):
        """work: the all-reduce of this gradient, still to be waited for.  The update stream waits for it (the
        collective itself was ordered after the gradient's producer when it was launched); without a collective the
        update stream forks from the calling stream here."""
        if not self._overlapping():
            if work is not None:
                work.wait()
            return self._update_param(p, group, pack)
        side, main = self.update_stream(p.device), torch.cuda.current_stream(p.device)
        if work is None or not self.__dict__.get("_forked"):
            side.wait_stream(main)
        with torch.cuda.stream(side):
            if work is not None:
                work.wait()
            self._update_param(p, group, pack)
        # gradients were allocated on the capturing stream and die with this call: keep their memory out of reuse
        # until the update that reads them has run
        for t in (*(pack or ()), p.grad):
            if torch.is_tensor(t) and t.is_cuda:
                t.record_stream(side)
        published = getattr(p, "_v4_scale", None)
        if published is not None and published[2] == side.cuda_stream:
            p._v4_scale = (published[0], published[1], main.cuda_stream, published[3])
        self.__dict__.setdefault("_forked", set()).add(torch.device(p.device).index)

    def _join_updates(self):
        for index in self.__dict__.pop("_forked", ()):
            torch.cuda.current_stream(index).wait_stream(self._update_streams[index])

    def _publish_scale(self, p, scale):
        p._v4_scale = (p._version, p.data_ptr(), torch.cuda.current_stream(p.device).cuda_stream, scale)

    def _update_param(self, p, g, pack=None):
        """Base path: FP32 master; compact INT8 m + FP16 v (format tile32) or plain FP32 moments for small tensors."""
        n = p.numel()
        compact = g['compact'] and n >= 4096
        s = self._state_for(p, g)
        ctrl = getattr(self, "_graph_control", None)
        t = s['step'] + 1
        cache = g['cache_scale'] and getattr(p, '_v4_request_scale', False)
        grad, sa, sb = pack if pack is not None else (p.grad, None, None)
        with torch.cuda.device(p.device):
            if compact:
                scale = None
                if cache:
                    scale = getattr(p, "_v5_graph_scale", None)
                    if scale is None:
                        scale = torch.empty((), device=p.device, dtype=torch.float32)
                scaled = pack is not None and sa is not None
                nat.adamw_step(p, 32, grad, s['m'], s['v'], s['ms'], s['vs'], vbits=16, mbits=8, nonlinear_m=False, state_block=BLOCK,
                               hyper=self._hyper(g, t), step=t, key=0, grad_kind=2 if scaled else None,
                               grad_cols=p.shape[-1] if scaled else 1, grad_stride=grad.shape[-1] if scaled else 1, sa=sa, sb=sb,
                               extra=p.grad if (pack is not None and p.grad is not None) else None, grad_mul=self._grad_mul(),
                               ctrl=ctrl, scale_out=scale)
                torch.autograd.graph.increment_version(p)
                if cache:
                    self._publish_scale(p, scale)
            else:
                if pack is not None:
                    raise RuntimeError("Deferred gradients need the compact update path")
                gr = grad if grad.dtype == torch.float32 else grad.float()
                nat.adamw_plain(p, gr.contiguous(), s['m'], s['v'], hyper=self._hyper(g, t), grad_mul=self._grad_mul(), ctrl=ctrl)
                torch.autograd.graph.increment_version(p)
            s['step'] = t

    # ---- eager entry points --------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, closure=None):
        self._require_eager()
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        active = [(p, g) for g in self.param_groups for p in g['params'] if p.grad is not None]
        if any(not p.is_contiguous() or p.grad.is_sparse or not p.grad.is_contiguous() for p, g in active):
            raise ValueError('Dense contiguous parameters and gradients required')
        if self.reducer is not None:
            self.reducer.begin([p for p, _ in active])     # an eager step: nothing is streamed, every collective is waited for
            self.reducer.reduce_dense([p for p, _ in active])
        for p, g in active:
            self._update_param(p, g)
        return loss

    def _owners(self, params):
        return [p for p, _ in params if getattr(p, "_v4_request_scale", False) or getattr(p, "_v6_defer_dense", False)]

    def backward_step(self, loss, *, audit=False):
        """Single eager backward + update.  Call zero_grad(set_to_none=True) first.  Converted layers leave their
        weight gradient in GEMM-output form for the update kernel; other contributions are added in FP32."""
        self._require_eager()
        params = [(p, g) for g in self.param_groups for p in g["params"]]
        pending = {}
        owners = self._owners(params)
        if any(p.grad is not None for p, _ in params):
            raise RuntimeError("backward_step requires cleared gradients")
        if any(hasattr(p, "_v4_pending") or p._backward_hooks or p._post_accumulate_grad_hooks for p in owners):
            raise RuntimeError("Gradient hooks or nested backward_step require ordinary backward/step")
        reducer = self.reducer
        try:
            for p in owners:
                p._v4_pending = pending
                if reducer is not None:
                    p._dp_reducer = reducer
            if reducer is not None:
                reducer.begin([p for p, _ in params])
            loss.backward()
        finally:
            for p in owners:
                del p._v4_pending
                if hasattr(p, "_dp_reducer"):
                    del p._dp_reducer
        active = [(p, g) for p, g in params if p in pending or p.grad is not None]
        for p, _ in active:
            if (not p.is_cuda or p.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn)
                    or not p.is_contiguous() or (p.grad is not None and (p.grad.is_sparse or not p.grad.is_contiguous()))):
                raise ValueError("Expected contiguous CUDA FP32 parameters and dense gradients")
        if reducer is not None:
            # every gradient autograd left in .grad, also the second gradient of a parameter whose first one sits in a
            # reducer slot (a weight shared with an embedding, a layer applied twice)
            reducer.finish([p for p, _ in active])
        if audit:
            checks = [torch.isfinite(p.grad).all() for p, _ in active if p.grad is not None]
            checks.extend(torch.isfinite(t).all() for pack in pending.values() for t in pack if torch.is_tensor(t))
            if not torch.stack(checks).all().item():
                raise RuntimeError("Nonfinite gradient before update")
        with torch.no_grad():
            for p, g in active:
                self._update_param(p, g, pending.pop(p, None))

    def _finish_streamed(self, p, group, pack, held, work=None):
        """Update p from a gradient whose all-reduce has completed (stream-wise)."""
        grad = held.pop(p, None)
        deferred = pack is not None and (pack[1] is not None or self.reducer.has_slot(p))
        if not deferred:
            # dense leaf gradient (reduced in place, or a view of a reduced bucket): the ordinary path reads p.grad
            p.grad = pack[0] if pack is not None else grad
            self._update_overlapped(p, group, None, work)
        else:
            p.grad = grad      # None, or a second gradient beside the deferred one: the update adds it in FP32
            self._update_overlapped(p, group, pack, work)
        p.grad = None

    def capture_streaming_backward(self, loss):
        """Record parameter-local updates once, as soon as each parameter's gradient is complete, inside backward
        (peak memory = one layer's gradient).  Only valid while a CUDA graph is being captured."""
        if not torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Streaming updates are available only during graph capture")
        params = [(p, g) for g in self.param_groups for p in g["params"]]
        storages = [p.untyped_storage().data_ptr() for p, g in params]
        if len(set(storages)) != len(storages):
            raise ValueError("Distinct optimizer entries may not alias storage")
        if any(p.grad is not None or p._backward_hooks or p._post_accumulate_grad_hooks for p, g in params):
            raise ValueError("Clear gradients and remove gradient hooks before capture")
        pending, completed, handles, held = {}, set(), [], {}
        owners = self._owners(params)
        reducer = self.reducer

        def ready(p, group):
            def update(grad_inputs, grad_outputs):
                pack = pending.pop(p, None)
                if p in completed or (pack is None and p.grad is None):
                    raise RuntimeError("Unexpected leaf gradient during capture")
                with torch.no_grad():
                    if reducer is None:
                        self._update_overlapped(p, group, pack)
                        p.grad = None
                    else:
                        held[p] = p.grad          # keep the leaf gradient alive until its collective is consumed
                        p.grad = None
                        both = pack is not None and held[p] is not None
                        for q, gq, packq, work in reducer.submit(p, group, pack if pack is not None else (held[p], None, None),
                                                                 wait=False, extra=held[p] if both else None):
                            self._finish_streamed(q, gq, packq, held, work)
                completed.add(p)
            return update
        try:
            for p in owners:
                p._v4_pending = pending
                if reducer is not None:
                    p._dp_reducer = reducer
            if reducer is not None:
                reducer.begin([p for p, _ in params], capturing=True)
            for p, group in params:
                node = torch.autograd.graph.get_gradient_edge(p).node
                handles.append(node.register_hook(ready(p, group)))
            loss.backward()
            if reducer is not None:
                with torch.no_grad():
                    for q, gq, packq, work in reducer.drain(wait=False):
                        self._finish_streamed(q, gq, packq, held, work)
            if pending or len(completed) != len(params):
                raise RuntimeError("Every parameter must receive its complete gradient once")
        finally:
            self._join_updates()
            for handle in handles:
                handle.remove()
            for p in owners:
                del p._v4_pending
                if hasattr(p, "_dp_reducer"):
                    del p._dp_reducer


class AdamW6(AdamW):
    """The storage formats of the six profiles: master in FP32 / FP16 / BF16(+tail) / E4M3 x unit, 8- or 4-bit moments."""

    def __init__(self, params, fmt, lr=1e-4, tiles=4, warps=4, **kw):
        super().__init__(params, lr=lr, **kw)
        for group in self.param_groups:
            group.update(format=fmt, tiles=tiles, warps=warps, state_block=state_block(fmt))
        self.keys = {p: 12345 + 7919 * i for i, p in enumerate(p for g in self.param_groups for p in g['params'])}

    def _state_for(self, p, g):
        if p.numel() < 4096 or not g['compact']:
            return super()._state_for(p, g)
        _, vb, mb = FORMATS[g['format']]
        s = self.state[p]
        if 'm' not in s:
            n = p.numel()
            s.update(step=0,
                     m=torch.zeros((n + 1) // 2 if mb == 4 and vb != 4 else n, device=p.device, dtype=torch.uint8 if mb == 4 else torch.int8),
                     ms=torch.zeros(cdiv(n, 64 if mb == 4 else g["state_block"]), device=p.device, dtype=torch.float32),
                     vs=torch.zeros(cdiv(n, 64 if vb == 4 else g["state_block"]), device=p.device, dtype=torch.float32))
            if vb != 4 or mb != 4:
                s['v'] = torch.zeros(cdiv(n, 2) if vb == 4 else n, device=p.device, dtype=torch.uint8 if vb < 16 else torch.float16)
        return s

    def _update_param(self, p, g, pack=None, sparse=None):
        n = p.numel()
        if n < 4096 or not g['compact']:
            return super()._update_param(p, g, pack)
        if sparse is not None:
            raise NotImplementedError("compact tied-embedding updates are not part of this interface")
        master, vb, mb = FORMATS[g['format']]
        if p.dtype == torch.float32:
            master = 32
        s = self._state_for(p, g)
        ctrl = getattr(self, '_graph_control', None)
        t = s['step'] + 1
        cache = g['cache_scale'] and getattr(p, '_v4_request_scale', False)
        grad, sa, sb = pack if pack is not None else (p.grad, None, None)
        scaled = pack is not None and sa is not None
        scale = None
        if cache:
            scale = getattr(p, '_v5_graph_scale', None)
            if scale is None:
                scale = torch.empty((), device=p.device, dtype=torch.float32)
        store = p.view(torch.uint8) if p.dtype == torch.float8_e4m3fn else p
        if not scaled and grad.dtype not in (torch.float32, torch.bfloat16):
            grad = grad.float()   # FP16 leaf gradients of FP16 masters: exact widening
        nonlinear = g['format'].endswith('_sqrt')
        emit = getattr(p, '_v6_pack', None)
        if emit is not None and cache and p.ndim == 2 and (master, vb, mb, nonlinear, g['state_block']) in nat.PREPACK_FORMATS:
            # one launch: the update, the next tensor scale and both packings of the updated weight
            nat.adamw_step_prepack(store, master, grad, s['m'], s.get('v'), s['ms'], s['vs'], pack=emit['buffers'], vbits=vb, mbits=mb,
                                   nonlinear_m=nonlinear, state_block=g['state_block'], hyper=self._hyper(g, t), step=t,
                                   key=self.keys[p], grad_kind=2 if scaled else None, grad_cols=p.shape[-1] if scaled else 1,
                                   grad_stride=grad.shape[-1] if scaled else 1, sa=sa, sb=sb,
                                   extra=p.grad if (pack is not None and p.grad is not None) else None, grad_mul=self._grad_mul(),
                                   tail=s.get('tail'), ctrl=ctrl, scale_out=scale)
            torch.autograd.graph.increment_version(p)
            emit['version'] = p._version
            s['step'] = t
            self._publish_scale(p, scale)
            self.prepacked = getattr(self, 'prepacked', 0) + 1
            return
        nat.adamw_step(store, master, grad, s['m'], s.get('v'), s['ms'], s['vs'], vbits=vb, mbits=mb,
                       nonlinear_m=g['format'].endswith('_sqrt'), state_block=g['state_block'], hyper=self._hyper(g, t), step=t,
                       key=self.keys[p], grad_kind=2 if scaled else None, grad_cols=p.shape[-1] if scaled else 1,
                       grad_stride=grad.shape[-1] if scaled else 1, sa=sa, sb=sb,
                       extra=p.grad if (pack is not None and p.grad is not None) else None, grad_mul=self._grad_mul(),
                       tail=s.get('tail'), unit=getattr(p, '_v6_unit', None), ctrl=ctrl, scale_out=scale)
        torch.autograd.graph.increment_version(p)
        s['step'] = t
        if cache:
            self._publish_scale(p, scale)

    def load_state_dict(self, state_dict):
        if any(a['format'] != b['format'] for a, b in zip(self.param_groups, state_dict['param_groups'])):
            raise ValueError('Checkpoint and model storage formats differ')
        return super().load_state_dict(state_dict)
