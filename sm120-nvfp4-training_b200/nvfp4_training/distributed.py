"""Data-parallel training: replicas that all-reduce weight gradients over NCCL (NVLink / NVSwitch).

The reference is single-GPU; this module is new.  Design:
  * every converted layer owns a persistent flat BF16 gradient slot; the wgrad GEMM's epilogue writes the scaled
    gradient straight into it (no pack / copy kernel between GEMM and collective);
  * a slot is all-reduced asynchronously as soon as its layer's backward has produced it, in backward order, so the
    transfer overlaps the remaining backward compute (NCCL runs on its own stream; only the consumer waits);
  * the fused AdamW kernel reads the reduced slot in place and folds the 1/world_size into its gradient decode;
  * gradients that autograd leaves in .grad are reduced in FP32: large ones (embeddings) on their own, small ones (norm
    gains, biases) packed into buckets of `bucket_mb` megabytes, one collective per bucket;
  * stochastic-rounding seeds of gradient quantisation get a per-rank offset; weights are re-quantised locally and are
    identical on all ranks because weights, rounding keys and step numbers are.
Works eagerly and under CUDA-graph capture (the update of a parameter is deferred by `depth` parameters so that its
collective has time to finish).  Plain loads / NCCL only: no peer-memory kernels, no TMA multicast.

Failures are detected on the host, between steps, never by a kernel that waits for a peer:
  * `verify_layout` (run by enable_data_parallel): every rank must hold the same slots, bucket size and depth, or all ranks
    raise before the first collective could pair buffers of different sizes;
  * `replica_digest` / `verify_replicas`: a SHA-256 over parameters, buffers and optimizer state; ranks that drifted apart
    (or loaded different checkpoints) raise on every rank, naming the ranks that disagree with rank 0;
  * `PeerWatch`: a gloo control group with a short timeout; `check()` before a step raises on the surviving ranks, naming
    the ranks that did not answer, instead of letting the next NCCL collective wait for a process that has left.
"""
from __future__ import annotations

import hashlib
from collections import deque
from datetime import timedelta

import torch
import torch.distributed as dist


class GradientReducer:
    def __init__(self, params, process_group=None, *, slot_dtype=torch.bfloat16, depth=2, owner_filter=None, bucket_mb=25.0):
        self.group = process_group
        self.world = dist.get_world_size(process_group)
        self.rank = dist.get_rank(process_group)
        self.grad_scale = 1.0 / self.world
        self.depth = max(0, int(depth))
        self.slot_dtype = slot_dtype
        self._slots = {}
        owners = [p for p in params if (owner_filter(p) if owner_filter else getattr(p, "_v4_request_scale", False))]
        for p in owners:
            self._slots[p] = torch.zeros(p.numel(), dtype=slot_dtype, device=p.device)
        self._works = []          # eager mode: outstanding collectives
        self._queue = deque()     # capture / streaming mode: (param, group, pack, work) waiting for their collective
        self.launched = []        # order in which slots were reduced (introspection / tests)
        self._streaming = False   # True between begin(capturing=True) and the next begin()
        self.bucket_bytes = int(float(bucket_mb or 0) * 2 ** 20)
        self._bucket = []         # (param, group, gradient) of small dense gradients waiting for a shared collective
        self._bucket_fill = 0
        self.collectives = 0      # collectives started since begin()
        self.elide = False        # timing experiments only: record no collective at all (results are then wrong on purpose)

    # ---- used by the linear layer's backward ------------------------------------------------------------
    def has_slot(self, p) -> bool:
        return p in self._slots

    def slot(self, p) -> torch.Tensor:
        return self._slots[p]

    def ready(self, p):
        """The slot of p holds this rank's gradient: start its all-reduce (eager mode)."""
        if self._streaming:
            return
        self._works.append(dist.all_reduce(self._slots[p], group=self.group, async_op=True))
        self.launched.append(p)

    # ---- eager protocol (backward_step / step) ----------------------------------------------------------
    def begin(self, params, capturing=False):
        watch = getattr(self, "watch", None)
        if watch is not None and not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()):
            watch.check()
        self._streaming = bool(capturing)
        self._works.clear()
        self._queue.clear()
        self.launched.clear()
        self._bucket.clear()
        self._bucket_fill = 0
        self.collectives = 0

    def finish(self, dense_params):
        """Reduce the gradients autograd left in .grad, then wait (stream-wise) for every collective."""
        self.reduce_dense(dense_params)
        for work in self._works:
            work.wait()
        self._works.clear()

    def reduce_dense(self, params):
        """All-reduce the gradients autograd left in .grad and wait for them (stream-wise)."""
        for p in params:
            if p.grad is not None:
                self._works.append(dist.all_reduce(p.grad, group=self.group, async_op=True))
        for work in self._works:
            work.wait()
        self._works.clear()

    # ---- streaming protocol (updates inside backward, eager or captured) ------------------------------
    def submit(self, p, group, pack, wait=True, extra=None):
        """Start the collective for p's gradient and return the (param, group, pack) items whose collectives have had
        `depth` later submissions to overlap with; those are safe to update now (after a stream-level wait).
        wait=False leaves that wait to the caller, who gets (param, group, pack, work) and may place it on the stream
        its update runs on, so that the calling stream never waits for a collective.
        extra: a second gradient of the same parameter that autograd left in .grad (a weight shared with an embedding, a
        layer applied twice); it is reduced as well and the returned work waits for both.
        A dense gradient of at most a quarter of a bucket joins the open bucket instead of getting its own collective."""
        tensor = pack[0] if pack is not None else p.grad
        dense = pack is None or (pack[1] is None and pack[2] is None and not self.has_slot(p))
        nbytes = tensor.numel() * 4
        if dense and extra is None and self.bucket_bytes and nbytes * 4 <= self.bucket_bytes:
            self._bucket.append((p, group, tensor))
            self._bucket_fill += nbytes
            self.launched.append(p)
            if self._bucket_fill >= self.bucket_bytes:
                self._flush_bucket()
            return self._pop(self.depth, wait)
        work = self._all_reduce(tensor)
        if extra is not None:
            work = _Both(work, self._all_reduce(extra))
        self.launched.append(p)
        self._queue.append(([(p, group, pack)], work))
        return self._pop(self.depth, wait)

    def _all_reduce(self, tensor):
        self.collectives += 1
        if self.elide:
            return _Done()
        return dist.all_reduce(tensor, group=self.group, async_op=True)

    def _flush_bucket(self):
        """One FP32 buffer, one collective; the members' gradients become views of the reduced buffer."""
        if not self._bucket:
            return
        flat = torch.cat([t.reshape(-1).float() for _, _, t in self._bucket])
        work = self._all_reduce(flat)
        items, at = [], 0
        for p, group, t in self._bucket:
            items.append((p, group, (flat[at:at + t.numel()].view(t.shape), None, None)))
            at += t.numel()
        self._queue.append((items, work))
        self._bucket.clear()
        self._bucket_fill = 0

    def drain(self, wait=True):
        self._flush_bucket()
        return self._pop(0, wait)

    def _pop(self, keep, wait):
        ready = []
        while len(self._queue) > keep:
            items, w = self._queue.popleft()
            if wait:
                w.wait()
                ready.extend(items)
            else:
                ready.extend((q, g, k, w) for q, g, k in items)
        return ready


    def layout(self):
        """What has to agree across ranks for the collectives to pair up: slot sizes in order, bucket size, depth."""
        return (tuple(t.numel() for t in self._slots.values()), str(self.slot_dtype), self.bucket_bytes, self.depth)


def _gather(value, group):
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, value, group=group)
    return out


def verify_layout(reducer):
    """Raise ValueError on EVERY rank when the ranks' reducers would pair buffers of different sizes."""
    layouts = _gather(reducer.layout(), reducer.group)
    odd = [r for r, l in enumerate(layouts) if l != layouts[0]]
    if odd:
        raise ValueError(f"Data-parallel ranks disagree on gradient slots, bucket size or depth: ranks {odd} differ from rank 0")


def replica_digest(model, optimizer=None):
    """SHA-256 over every parameter and buffer (and, when given, every tensor of the optimizer state) in registration
    order: equal on all ranks of a healthy data-parallel job after any number of steps."""
    h = hashlib.sha256()

    def feed(t):
        t = t.detach()
        raw = t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t
        h.update(str((tuple(t.shape), str(t.dtype))).encode())
        h.update(raw.contiguous().cpu().reshape(-1).view(torch.uint8).numpy().tobytes())

    for _, t in list(model.named_parameters()) + list(model.named_buffers()):
        feed(t)
    if optimizer is not None:
        for group in optimizer.param_groups:
            for p in group["params"]:
                for key, value in sorted(optimizer.state.get(p, {}).items(), key=lambda kv: str(kv[0])):
                    if torch.is_tensor(value):
                        feed(value)
                    else:
                        h.update(repr((key, value)).encode())
    return h.hexdigest()


def verify_replicas(model, optimizer=None, process_group=None):
    """Compare replica_digest across ranks; RuntimeError on every rank when they differ.  Call between steps (it copies
    the state to the host), e.g. after loading a checkpoint on every rank and before writing one."""
    digests = _gather(replica_digest(model, optimizer), process_group)
    odd = [r for r, d in enumerate(digests) if d != digests[0]]
    if odd:
        raise RuntimeError(f"Data-parallel replicas diverged: ranks {odd} hold different state than rank 0")
    return digests[0]


class PeerWatch:
    """Host-side liveness check over a gloo control group: `check()` returns when every rank reached it within the
    timeout and raises RuntimeError naming the missing ranks otherwise.  A rank leaves a job only between steps; the
    others call check() before their next launch, so no kernel or NCCL collective ever waits for a process that is gone."""

    def __init__(self, timeout_s=30.0, ranks=None):
        self.timeout = timedelta(seconds=float(timeout_s))
        self.group = dist.new_group(ranks=ranks, backend="gloo", timeout=self.timeout)

    def check(self):
        try:
            dist.monitored_barrier(group=self.group, timeout=self.timeout, wait_all_ranks=True)
        except RuntimeError as e:
            raise RuntimeError(f"Data-parallel peer check failed before the step: {e}") from e


class _Done:
    def wait(self):
        pass


class _Both:
    """Two collectives that one update waits for."""

    def __init__(self, first, second):
        self.first, self.second = first, second

    def wait(self):
        self.first.wait()
        self.second.wait()


def enable_data_parallel(model, process_group=None, *, bucket_mb=25.0, depth=2, peer_timeout=None):
    """Attach a GradientReducer to model.nvfp4_optimizer.  Call after enable_nvfp4 on every rank; rank 0's weights are
    broadcast.  The process group defaults to the world group.  depth: how many later gradients' collectives are started
    before an update waits for its own (captured steps).  bucket_mb: small dense gradients (norm gains, biases) share
    FP32 buckets of this size, one collective each; the weight gradients of converted layers are 19 MB and more each and
    keep their own collective, written in place by the weight-gradient GEMM (0 gives every gradient its own).
    peer_timeout: seconds; when given, a PeerWatch is attached as `reducer.watch` and checked at the start of every eager
    step (call `reducer.watch.check()` yourself between replays of a captured step)."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialised before enable_data_parallel")
    opt = model.nvfp4_optimizer
    params = [p for g in opt.param_groups for p in g["params"]]
    if process_group is None and dist.get_backend() == "nccl" and getattr(opt, "overlap_updates", False):
        # A captured step runs its main line on a high-priority stream and the optimizer updates below it; the
        # collectives belong with the main line, or they would only run in its gaps and pile up behind backward.
        options = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        process_group = dist.new_group(ranks=list(range(dist.get_world_size())), backend="nccl", pg_options=options)
    reducer = GradientReducer(params, process_group, depth=depth, bucket_mb=bucket_mb)
    verify_layout(reducer)
    reducer.watch = PeerWatch(peer_timeout) if peer_timeout else None
    opt.reducer = reducer
    from ._backend import quant
    quant._RANK_OFFSET = (reducer.rank * 0x9E3779B1) & 0xFFFFFFFF
    # replicas must start from identical weights
    with torch.no_grad():
        for p in params:
            src = p.view(torch.uint8) if p.dtype == torch.float8_e4m3fn else p
            dist.broadcast(src, src=dist.get_global_rank(process_group, 0) if process_group is not None else 0, group=process_group)
        for b in model.buffers():
            if b.is_floating_point() or b.dtype in (torch.uint8, torch.int8):
                dist.broadcast(b, src=dist.get_global_rank(process_group, 0) if process_group is not None else 0, group=process_group)
    return model
