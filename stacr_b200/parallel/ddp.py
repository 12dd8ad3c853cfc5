"""Data-parallel gradient synchronisation with rank-local compression state.

``GradSync`` owns one flat fp32 gradient buffer; every ``param.grad`` is a view into it, so
gradients are produced in place, reduced in place and consumed in place by the fused optimizer.
Parameters are grouped into buckets in reverse registration order (the order backward produces
them).  A post-accumulate hook marks a parameter ready; when a bucket is complete its slice is
averaged across ranks on a communication stream while backward keeps running.  The reduction
itself is pluggable:

* ``"symm"``: the in-tree all-reduce kernels over NVLink peer memory / NVSwitch multimem
  (``stacr_b200.parallel.symm``), used on CUDA when symmetric memory is available;
* ``"nccl"`` / ``"gloo"``: ``torch.distributed.all_reduce`` (the portable path; also what the
  CPU tests run with two gloo ranks).

Bases, step counters and residual state of the compressed layers are *not* synchronised: each
rank tracks the subspace of its own data shard, as the reference prescribes for DDP
(``broadcast_buffers=False``; experiments/protocols/training.py:507-509 there).
"""

from __future__ import annotations

import contextlib

import os
import weakref
from typing import Iterable

import torch
import torch.distributed as dist
from torch import nn


def init_distributed(backend: str | None = None) -> tuple[int, int, int]:
    """Initialise the default process group from torchrun's environment; returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, world, local


def broadcast_parameters(model: nn.Module, src: int = 0) -> None:
    """Make every rank start from rank ``src``'s parameters (buffers stay rank-local)."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return
    for p in model.parameters():
        # through ``detach()`` (shares the version counter), not ``.data``: a cached bf16 shadow of the parameter is
        # keyed on that counter and must see this write
        with torch.no_grad():
            dist.broadcast(p.detach(), src)


class GradSink:
    """Where a compressed layer's weight-gradient kernel delivers its result (see ``ops.stacr_ops.weight_grad``).

    ``mode`` 1 adds into this rank's flat buffer; ``mode`` 2 adds each 16-byte element into the copy of the rank that
    owns its slice of the parameter's slot (the reduce-scatter half of the all-reduce, done inside the kernel over
    NVLink peer memory).  ``done()`` tells the synchroniser that the parameter's contribution is enqueued.
    """

    def __init__(self, sync: "GradSync", index: int, offset: int, numel_padded: int):
        self.sync, self.index = sync, index
        self.flat = sync.flat
        self.param_off = offset
        self.region_lo = offset
        self.region_hi = offset + numel_padded
        self.world = sync.world
        self.scale = 1.0
        if sync.backend == "symm":
            self.mode = 2
            self.per_vecs = sync._symm.slice_vecs(offset, offset + numel_padded)
            self.peer_ptrs = sync._symm.peer_ptrs
        else:
            self.mode, self.per_vecs, self.peer_ptrs = 1, 1, None

    def done(self) -> None:
        self.sync._fused_done(self.index)


class GradSync:
    """Flat-buffer, bucketed, overlapped gradient averaging for one model replica.

    ``fused`` names parameters (the weights of compressed layers) whose gradient kernel writes into the flat buffer
    itself: they get a :class:`GradSink` as ``param._sb_grad_sink``, are left out of the hook-driven buckets, and are
    finished by an all-gather of owner slices (symmetric-memory backend) or one all-reduce (other backends).
    """

    def __init__(self, params: Iterable[nn.Parameter], *, bucket_mb: float = 256.0, backend: str = "auto",
                 group=None, average: bool = True, fused: Iterable[nn.Parameter] = (), heartbeat=None):
        self.heartbeat = heartbeat      # optional health.Heartbeat: peers' failures raise here, ours is published to them
        fused_ids = {id(p) for p in fused if p.requires_grad}
        ordered = [p for p in params if p.requires_grad]
        # fused parameters first: their slots form the head of the flat buffer
        self.params = [p for p in ordered if id(p) in fused_ids] + [p for p in ordered if id(p) not in fused_ids]
        self.n_fused = sum(1 for p in self.params if id(p) in fused_ids)
        if not self.params:
            raise ValueError("GradSync needs at least one trainable parameter")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.average = average
        dev = self.params[0].device
        self.device = dev
        total = sum(p.numel() for p in self.params)
        # pad each parameter's slot to 16 bytes so every view is vector-aligned
        offsets, cursor = [], 0
        for p in self.params:
            offsets.append(cursor)
            cursor += (p.numel() + 3) // 4 * 4
        self.numel = cursor
        self.backend = self._pick_backend(backend, dev)
        self.flat = self._allocate(cursor, dev)
        self.flat.zero_()
        self._views = [self.flat[off:off + p.numel()].view_as(p) for p, off in zip(self.params, offsets)]
        for p, view in zip(self.params, self._views):
            p.grad = view
            p._sb_grad_out = view          # layers write their first gradient of a step straight into the slot ...
            p._sb_grad_fresh = False
        self._written = [True] * len(self.params)
        self._counted = [False] * len(self.params)
        # buckets over the reversed parameter list (backward order)
        limit = int(bucket_mb * 1024 * 1024 / 4)
        self.buckets: list[tuple[int, int]] = []
        self._members: list[list[int]] = []
        self._bucket_of: dict[int, int] = {}
        self._pending: list[int] = []
        hi = cursor
        lo = hi
        members: list[int] = []
        for idx in range(len(self.params) - 1, self.n_fused - 1, -1):
            lo = offsets[idx]
            members.append(idx)
            if hi - lo >= limit or idx == self.n_fused:
                b = len(self.buckets)
                self.buckets.append((lo, hi))
                self._members.append(list(members))
                for m in members:
                    self._bucket_of[m] = b
                self._pending.append(len(members))
                members, hi = [], lo
        self._size = list(self._pending)
        self._stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self._launched = 0
        self.reductions = 0
        self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(i)) for i, p in enumerate(self.params)]
        for i, p in enumerate(self.params):
            if i >= self.n_fused:
                p._sb_grad_ready = self._make_ready(i)     # ... and then call this instead of returning the gradient to autograd
        self._total = total
        self._offsets = offsets
        self._syncing = True
        self.sinks: list[GradSink] = []
        self._fused_state = [0] * self.n_fused       # 0 idle, 1 delivered by the kernel, 2 accumulated by autograd
        for i in range(self.n_fused):
            p = self.params[i]
            sink = GradSink(self, i, offsets[i], (p.numel() + 3) // 4 * 4)
            p._sb_grad_sink = sink
            self.sinks.append(sink)

    # ------------------------------------------------------------------ backend plumbing
    def _pick_backend(self, backend: str, dev: torch.device) -> str:
        if self.world == 1:
            return "none"
        if backend != "auto":
            return backend
        if dev.type == "cuda":
            from . import symm

            return "symm" if symm.available() else "nccl"
        return "gloo"

    def _allocate(self, numel: int, dev: torch.device) -> torch.Tensor:
        if self.backend == "symm":
            from . import symm

            self._symm = symm.SymmetricBuffer(numel, torch.float32, dev, self.group)
            return self._symm.tensor
        return torch.empty(numel, dtype=torch.float32, device=dev)

    def _reduce(self, lo: int, hi: int) -> None:
        if self.backend == "none" or hi <= lo:
            return
        self.reductions += 1
        if self.backend == "symm":
            self._symm.all_reduce_(lo, hi, average=self.average)
            return
        chunk = self.flat[lo:hi]
        dist.all_reduce(chunk, op=dist.ReduceOp.SUM, group=self.group)
        if self.average:
            chunk.div_(self.world)

    # ------------------------------------------------------------------ hooks
    def _make_hook(self, index: int):
        # The hook is owned by the tensor's C++ autograd state, which Python's cycle collector cannot see through: a hook that
        # held this object strongly would tie it (and the flat buffer, and every parameter) to the parameters for ever.
        ref = weakref.ref(self)
        if index < self.n_fused:
            def fused_hook(param):
                me = ref()
                if me is None:
                    return
                me._adopt(index, param)
                me._fused_state[index] = 2      # autograd accumulated a dense gradient locally (layer ran uncompressed)
            return fused_hook

        def hook(param):
            me = ref()
            if me is None:
                return
            me._written[index] = True         # moved into its slot together with the rest of its bucket
            if not me._syncing or me._counted[index]:
                return                        # a layer that handed its slot over directly has already been counted this pass
            me._counted[index] = True
            b = me._bucket_of[index]
            me._pending[b] -= 1
            if me._pending[b] == 0:
                me._launch(b)
        return hook

    def _make_ready(self, index: int):
        """Hand-over used by layers that have written a parameter's gradient into its slot themselves.

        Returning the slot to autograd would not do: the engine clones a gradient that anything else still references
        (the slot is referenced from here), and the clone would then be copied back.  The layer instead writes the slot,
        calls this, and returns no gradient for the parameter.  Only valid for a parameter that receives one gradient per
        backward pass; tied parameters (``param._sb_tied``) keep the ordinary route.
        """
        hook = self._make_hook(index)

        def ready():
            param = self.params[index]
            param.grad = self._views[index]
            hook(param)
        return ready

    def _adopt_bucket(self, b: int) -> None:
        """Move the gradients of bucket ``b`` that autograd produced elsewhere into their slots with one multi-tensor copy."""
        src, dst = [], []
        for i in self._members[b]:
            p, view = self.params[i], self._views[i]
            g = p.grad
            if g is None:
                view.zero_()
            elif g.data_ptr() != view.data_ptr():
                src.append(g)
                dst.append(view)
            p.grad = view
            self._written[i] = True
        if src:
            torch._foreach_copy_(dst, src)

    def _launch(self, b: int) -> None:
        lo, hi = self.buckets[b]
        self._launched += 1
        self._adopt_bucket(b)
        if self.backend == "symm" and self._stream is not None:
            from ..ops import _lib

            if os.environ.get("STACR_COMM_RESERVE", "1") == "1":
                _lib.reserve_sms(self._symm.max_ctas)   # until finish(): the collectives of this step share the GPU with backward
        if self._stream is None:
            self._reduce(lo, hi)
            return
        self._stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._stream):
            self._reduce(lo, hi)

    def _adopt(self, index: int, param) -> None:
        """Make the parameter's gradient live in its slot of the flat buffer (a copy only if autograd produced it elsewhere)."""
        view = self._views[index]
        g = param.grad
        if g is not None and g.data_ptr() != view.data_ptr():
            view.copy_(g)
            param.grad = view
        self._written[index] = True

    # ------------------------------------------------------------------ fused parameters
    def _fused_done(self, index: int) -> None:
        if self._fused_state[index] == 0:
            self._fused_state[index] = 1
        if self._syncing and self.world > 1:
            self._finish_fused(index)

    def _finish_fused(self, index: int) -> None:
        state = self._fused_state[index]
        if state in (0, 3) or self.world == 1:
            return
        sink = self.sinks[index]
        self._fused_state[index] = 3
        self.reductions += 1
        cur = torch.cuda.current_stream(self.device) if self._stream is not None else None
        if cur is not None:
            self._stream.wait_stream(cur)
        ctx = torch.cuda.stream(self._stream) if self._stream is not None else contextlib.nullcontext()
        with ctx:
            if self.backend == "symm" and state == 1:
                self._symm.all_gather_slices_(sink.region_lo, sink.region_hi, average=self.average)
            else:
                self._reduce(sink.region_lo, sink.region_hi)
                self.reductions -= 1

    @contextlib.contextmanager
    def no_sync(self):
        """Gradient accumulation: backward passes inside do not start reductions; ``finish()`` after the last one does."""
        self._syncing = False
        try:
            yield
        finally:
            self._syncing = True

    # ------------------------------------------------------------------ step protocol
    def zero_grad(self) -> None:
        """Forget the gradients and re-arm the buckets.  Call instead of ``optimizer.zero_grad``.

        Nothing is cleared up front: every parameter's gradient is dropped (``grad = None``) so that autograd hands over
        its first gradient of the step instead of accumulating into zeros, and the hook moves it into the slot (or finds
        it already there when a compressed layer wrote the slot directly).  Slots that no backward pass touched are
        cleared in ``finish``.  The fused reduce-scatter path still needs zeros in every copy before any rank adds.
        """
        if self.n_fused:
            # slots that the gradient kernels add into (locally or from other ranks) must start from zero
            self.flat[: self.sinks[-1].region_hi].zero_()
            if self.backend == "symm":
                self._symm.barrier()   # no peer may add into this buffer before it is cleared
        for i, p in enumerate(self.params):
            if i < self.n_fused:
                p.grad = self._views[i]
                p._sb_grad_fresh = False
                self._written[i] = True
                continue
            p.grad = None
            p._sb_grad_fresh = True
            self._written[i] = False
        self._fused_state = [0] * self.n_fused
        self._pending = list(self._size)
        self._counted = [False] * len(self.params)
        self._launched = 0

    def finish(self) -> None:
        """Reduce buckets whose hooks did not all fire (unused parameters) and join the communication stream."""
        for b, left in enumerate(self._pending):
            if left > 0 or any(self.params[i].grad is None or self.params[i].grad.data_ptr() != self._views[i].data_ptr() for i in self._members[b]):
                self._pending[b] = 0
                self._launch(b)       # adopts (or clears) every slot of the bucket first
        for i in range(self.n_fused):
            if self._fused_state[i] == 0 and self.backend == "symm":
                self._fused_state[i] = 1   # unused this step on this rank: peers may still have added into our slice
            self._finish_fused(i)
        if self._stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._stream)
        if self.backend == "symm":
            from ..ops import _lib

            _lib.reserve_sms(0)
        self.check_health()

    def check_health(self) -> None:
        """Raise on every rank when a collective of this or the previous step gave up waiting for a peer.

        The in-tree collectives bound every wait; a rank that times out records a code in its device status word and
        returns without having reduced.  The word is read here once per step through a pinned asynchronous copy (one
        step late, no host wait; synchronously under ``STACR_STRICT_STATUS=1``), so un-averaged gradients are applied for
        at most one step before ``KernelError`` stops the job.  A peer's ``RankFailure`` recorded in the job store by
        ``health.Heartbeat`` is raised by the heartbeat's own ``check``.
        """
        if self.heartbeat is not None:
            self.heartbeat.check()          # a peer that failed or left: stop before its missing contribution is applied again
        if self.device.type != "cuda":
            return
        from ..ops import _lib

        try:
            _lib.poll_status(self.device)
        except _lib.KernelError as exc:
            if self.heartbeat is not None:
                self.heartbeat.fail(f"KernelError: {exc}")   # the other ranks raise RankFailure at their next check
            raise

    def close(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
        for p in self.params:
            for attr in ("_sb_grad_sink", "_sb_grad_out", "_sb_grad_fresh", "_sb_grad_ready"):
                if hasattr(p, attr):
                    delattr(p, attr)


def all_reduce_mean_(tensor: torch.Tensor, group=None) -> torch.Tensor:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(tensor, group=group)
        tensor.div_(dist.get_world_size(group))
    return tensor
