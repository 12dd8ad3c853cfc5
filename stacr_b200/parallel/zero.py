"""Data parallelism with the optimizer sharded over the ranks (ZeRO stage 1), built for NVSwitch.

``ShardedGradSync`` keeps what ``GradSync`` does (one flat fp32 gradient buffer in symmetric memory, gradients produced
in place, buckets reduced on a communication stream while backward runs) and changes what is communicated:

* the large matrices (2-D parameters above ``shard_min_numel``) form the *sharded region*.  A bucket of it is only
  **reduced to its owners**: rank ``r`` sums slice ``r`` of the bucket over all ranks (``multimem.ld_reduce`` in the
  switch, or peer loads) and stores it in its own copy.  Nothing is broadcast, which halves the NVLink traffic of an
  all-reduce;
* each rank then runs the optimizer on the slices it owns, 1/W of the parameters, and the update kernel stores the new
  bf16 weights through the NVSwitch multicast address of a flat bf16 buffer that every rank's forward and backward
  read (``param._bf16_shadow`` views): the store of the optimizer *is* the all-gather.  A flag barrier behind the kernel
  makes the new weights visible everywhere before the next forward;
* everything else (biases, normalisation weights: a few MB) stays replicated: all-reduced and updated by every rank.

The fp32 master copy of a sharded matrix is current only on the owner of each slice; ``gather_parameters()`` makes all
copies current (call it before evaluating in fp32, checkpointing the model, or handing the model to other code).
Optimizer state exists for the whole model on every rank but is advanced only for the owned slices.

Without symmetric memory (NCCL on a fabric without multicast, gloo on CPU) the same partition is used with library
collectives: all-reduce of the bucket, and after the step an all-gather of the bf16 buffer (CUDA) or broadcasts of the
owned master slices (CPU, where there are no bf16 copies).

The reference trains data-parallel with DistributedDataParallel and a replicated optimizer
(experiments/benchmarks/distributed_data.py:87-97 there); this is the B200 form of the same job.
"""

from __future__ import annotations

import os
from typing import Iterable

import torch
import torch.distributed as dist
from torch import nn

from .ddp import GradSync

CHUNK = 2048      # elements per optimizer chunk: ownership boundaries fall on multiples of it relative to every parameter


class ShardedGradSync(GradSync):
    def __init__(self, params: Iterable[nn.Parameter], *, bucket_mb: float = 256.0, backend: str = "auto", group=None, average: bool = True,
                 shard_min_numel: int = 65536, heartbeat=None):
        self.heartbeat = heartbeat
        ordered = [p for p in params if p.requires_grad]
        if not ordered:
            raise ValueError("ShardedGradSync needs at least one trainable parameter")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.average = average
        dev = ordered[0].device
        self.device = dev
        self.backend = self._pick_backend(backend, dev)
        big = [p for p in ordered if p.dim() >= 2 and p.numel() >= shard_min_numel and p.numel() % 8 == 0 and p.dtype == torch.float32]
        big_ids = {id(p) for p in big}
        small = [p for p in ordered if id(p) not in big_ids]
        self.params = big + small
        self.n_sharded = len(big)
        self.n_fused, self.sinks, self._fused_state = 0, [], []
        # ---- layout.  Sharded region: buckets over the matrices in reverse registration order (the order backward
        # produces them); a parameter's slot starts on a chunk boundary and a bucket's length is a multiple of
        # CHUNK * world, so that the W equal slices of a bucket are whole chunks.
        limit = max(CHUNK * self.world, int(bucket_mb * 1024 * 1024 / 4))
        offsets = [0] * len(self.params)
        self.buckets: list[tuple[int, int]] = []
        self._members: list[list[int]] = []
        self._bucket_of: dict[int, int] = {}
        self._bucket_sharded: list[bool] = []
        cursor, start, members = 0, 0, []

        def close_bucket(sharded: bool):
            nonlocal cursor, start, members
            if not members:
                return
            if sharded:
                quantum = CHUNK * self.world
                cursor = start + (cursor - start + quantum - 1) // quantum * quantum
            b = len(self.buckets)
            self.buckets.append((start, cursor))
            self._members.append(list(members))
            self._bucket_sharded.append(sharded)
            for m in members:
                self._bucket_of[m] = b
            start, members = cursor, []

        for idx in range(self.n_sharded - 1, -1, -1):
            offsets[idx] = cursor
            cursor += (self.params[idx].numel() + CHUNK - 1) // CHUNK * CHUNK
            members.append(idx)
            if cursor - start >= limit:
                close_bucket(True)
        close_bucket(True)
        self.sharded_numel = cursor
        for idx in range(len(self.params) - 1, self.n_sharded - 1, -1):
            offsets[idx] = cursor
            cursor += (self.params[idx].numel() + 3) // 4 * 4
            members.append(idx)
        close_bucket(False)
        self.numel = cursor
        self._offsets = offsets
        self.flat = self._allocate(cursor, dev)
        self.flat.zero_()
        self._views = [self.flat[off:off + p.numel()].view_as(p) for p, off in zip(self.params, offsets)]
        for p, view in zip(self.params, self._views):
            p.grad = view
            p._sb_grad_out = view
            p._sb_grad_fresh = False
        self._written = [True] * len(self.params)
        self._counted = [False] * len(self.params)
        self._size = [len(m) for m in self._members]
        self._pending = list(self._size)
        self._stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self._launched = 0
        self.reductions = 0
        self._syncing = True
        self._total = sum(p.numel() for p in self.params)
        self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(i)) for i, p in enumerate(self.params)]
        for i, p in enumerate(self.params):
            p._sb_grad_ready = self._make_ready(i)
        # ---- ownership: slice `rank` of every sharded bucket
        self._owned: list[tuple[int, int]] = []
        for (lo, hi), sharded in zip(self.buckets, self._bucket_sharded):
            if sharded:
                per = (hi - lo) // self.world
                self._owned.append((lo + self.rank * per, lo + (self.rank + 1) * per))
        self._index = {id(p): i for i, p in enumerate(self.params)}
        # ---- the bf16 weights of the sharded region, one flat buffer laid out like the gradient buffer
        self._shadow = None
        self.shadow_flat = None
        if dev.type == "cuda" and self.n_sharded:
            try:
                self._make_shadows(dev)
            except Exception:
                # leave the parameters as they were found (hooks and gradient views gone), so that a caller can fall back to
                # the replicated path
                GradSync.close(self)
                raise

    # ------------------------------------------------------------------ bf16 weights
    def _make_shadows(self, dev) -> None:
        mc = 0
        if self.backend == "symm":
            from . import symm

            self._shadow = symm.SymmetricBuffer(self.sharded_numel, torch.bfloat16, dev, self.group)
            self.shadow_flat = self._shadow.tensor
            if self._shadow.use_multimem:
                mc = self._shadow.multicast_ptr
        else:
            self.shadow_flat = torch.empty(self.sharded_numel, dtype=torch.bfloat16, device=dev)
        self.shadow_flat.zero_()
        for i in range(self.n_sharded):
            p, off = self.params[i], self._offsets[i]
            view = self.shadow_flat[off:off + p.numel()].view_as(p)
            view.copy_(p.detach())
            p._bf16_shadow = view
            p._bf16_shadow_version = p._version
            p._bf16_shadow_mc = (mc + 2 * off) if mc else 0
        if self.backend == "symm":
            torch.cuda.synchronize(dev)
            dist.barrier(self.group)

    # ------------------------------------------------------------------ partition queries (used by the optimizer)
    def is_sharded(self, p: nn.Parameter) -> bool:
        i = self._index.get(id(p))
        return i is not None and i < self.n_sharded and self.world > 1

    def owned_ranges(self, p: nn.Parameter) -> list[tuple[int, int]]:
        """Element ranges of ``p`` (relative to its start, chunk aligned) that this rank's optimizer updates."""
        i = self._index[id(p)]
        if i >= self.n_sharded or self.world == 1:
            return [(0, p.numel())]
        off, n = self._offsets[i], p.numel()
        out = []
        for lo, hi in self._owned:
            a, b = max(lo, off), min(hi, off + n)
            if b > a:
                out.append((a - off, b - off))
        return out

    def owners_of(self, p: nn.Parameter) -> list[tuple[int, int, int]]:
        """``(rank, start, end)`` for every rank's part of ``p``."""
        i = self._index[id(p)]
        off, n = self._offsets[i], p.numel()
        out = []
        for (lo, hi), sharded in zip(self.buckets, self._bucket_sharded):
            if not sharded:
                continue
            per = (hi - lo) // self.world
            for r in range(self.world):
                a, b = max(lo + r * per, off), min(lo + (r + 1) * per, off + n)
                if b > a:
                    out.append((r, a - off, b - off))
        return out

    # ------------------------------------------------------------------ reductions
    def _reduce(self, lo: int, hi: int) -> None:
        if self.backend == "none" or hi <= lo:
            return
        self.reductions += 1
        b = next(i for i, (blo, bhi) in enumerate(self.buckets) if blo == lo and bhi == hi)
        if self.backend == "symm":
            if self._bucket_sharded[b]:
                per = (hi - lo) // self.world
                self._symm.reduce_to_owner_(lo, hi, lo + self.rank * per, lo + (self.rank + 1) * per, average=self.average)
            else:
                self._symm.all_reduce_(lo, hi, average=self.average)
            return
        chunk = self.flat[lo:hi]
        dist.all_reduce(chunk, op=dist.ReduceOp.SUM, group=self.group)
        if self.average:
            chunk.div_(self.world)

    # ------------------------------------------------------------------ after the optimizer step
    def publish_updates(self) -> None:
        """Make this step's new weights visible on every rank (called by the optimizer at the end of ``step``)."""
        if self.world == 1 or not self.n_sharded:
            return
        if self._shadow is not None and self._shadow.use_multimem:
            self._shadow.barrier()          # the update kernel stored through the multicast address: only ordering is left
            return
        if self.shadow_flat is not None:
            # library all-gather of the bf16 buffer, bucket by bucket (slice r of a bucket is rank r's)
            for (lo, hi), sharded in zip(self.buckets, self._bucket_sharded):
                if sharded:
                    per = (hi - lo) // self.world
                    dist.all_gather_into_tensor(self.shadow_flat[lo:hi], self.shadow_flat[lo + self.rank * per: lo + (self.rank + 1) * per],
                                                group=self.group)
            return
        self.gather_parameters()            # CPU: there are no bf16 copies, the masters themselves are exchanged

    @torch.no_grad()
    def gather_parameters(self) -> None:
        """Bring every rank's fp32 masters of the sharded matrices up to date (each slice comes from its owner)."""
        if self.world == 1:
            return
        for i in range(self.n_sharded):
            p = self.params[i]
            flat = p.detach().view(-1)
            for r, a, b in self.owners_of(p):
                dist.broadcast(flat[a:b], src=dist.get_global_rank(self.group, r) if self.group is not None else r, group=self.group)
            if hasattr(p, "_bf16_shadow_version"):
                p._bf16_shadow_version = p._version     # the bf16 copy already holds these values

    def close(self) -> None:
        super().close()
        for p in self.params:
            for attr in ("_bf16_shadow", "_bf16_shadow_version", "_bf16_shadow_mc"):
                if hasattr(p, attr):
                    delattr(p, attr)


def zero_enabled(default: bool = True) -> bool:
    """``STACR_ZERO=0/1`` overrides the caller's default for the sharded optimizer path."""
    value = os.environ.get("STACR_ZERO")
    return default if value is None else value == "1"
