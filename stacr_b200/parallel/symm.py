"""Symmetric peer memory and the in-tree all-reduce kernels over NVLink / NVSwitch.

Allocation and the peer-pointer exchange go through ``torch.distributed._symmetric_memory`` (CUDA
VMM allocations mapped into every rank of the node, plus an NVSwitch multicast address when the
fabric offers one).  The reductions are this framework's own kernels (``csrc/comm.cu``):

* two-shot all-reduce with plain peer loads/stores: each rank reduces its 1/W slice reading every
  peer's buffer, writes the result back to every peer; barriers are flag words in the symmetric
  signal pad with bounded waits;
* one-shot ``multimem.ld_reduce`` / ``multimem.st`` through the NVSwitch multicast address.

``available()`` is False when the build of PyTorch lacks symmetric memory or the process group is
not NCCL on CUDA; ``GradSync`` then uses the NCCL path.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib


def available() -> bool:
    if os.environ.get("STACR_DISABLE_SYMM", "0") == "1":
        return False
    if not (torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"):
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
    except Exception:
        return False
    return hasattr(_lib.load(), "sb_allreduce_two_shot")


class SymmetricBuffer:
    """A tensor that every rank of the group can address, with in-place all-reduce over its slices."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        # epoch-tagged barrier flags live in their own symmetric buffer
        self.flags = symm_mem.empty(_lib.load().sb_comm_flag_ints(), dtype=torch.int32, device=device)
        self.flags.zero_()
        self._flag_handle = symm_mem.rendezvous(self.flags, self.group)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # nobody may publish a flag before every rank has zeroed its own
        off = int(getattr(self.handle, "offset", 0) or 0)  # byte offset of the tensor inside its allocation
        foff = int(getattr(self._flag_handle, "offset", 0) or 0)
        ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
        pads = [int(p) + foff for p in self._flag_handle.buffer_ptrs]
        self._peer_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self._pad_ptrs = torch.tensor(pads, dtype=torch.int64, device=device)
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if self.multicast_ptr:
            self.multicast_ptr += off
        self.use_multimem = self.multicast_ptr != 0 and os.environ.get("STACR_SYMM_MULTIMEM", "1") == "1"
        self._epoch = 0
        # the barrier epoch lives on the device: a one-thread kernel advances it in front of every collective, which reads it
        # there.  A host-side counter passed by value would be frozen into a captured CUDA graph and break every replay.
        self._epoch_dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.numel = numel
        # CTAs per collective kernel: each one takes an SM away from the compute it overlaps with.  The switch-side
        # reduction (multimem) reaches its bandwidth with very few CTAs; peer loads/stores need many more in flight.
        self.max_ctas = int(os.environ.get("STACR_COMM_CTAS", "8" if self.use_multimem else "64"))

    def _next_epoch(self):
        """Advance the device-side epoch (stream-ordered) and return the ``(epoch, epoch_ptr)`` argument pair for the next kernel."""
        self._epoch += 1
        rc = _lib.load().sb_epoch_bump(_lib.ptr(self._epoch_dev), _lib.stream_ptr())
        _lib.check_rc(rc, "sb_epoch_bump")
        return ctypes.c_int(self._epoch), _lib.ptr(self._epoch_dev)

    def all_reduce_(self, lo: int, hi: int, average: bool = True) -> None:
        """In-place sum (or mean) of ``tensor[lo:hi]`` across ranks, on the current stream."""
        epoch = self._next_epoch()
        lib = _lib.load()
        scale = 1.0 / self.world if average else 1.0
        fn = lib.sb_allreduce_multimem if self.use_multimem else lib.sb_allreduce_two_shot
        rc = fn(
            _lib.ptr(self._peer_ptrs), _lib.ptr(self._pad_ptrs), ctypes.c_ulonglong(self.multicast_ptr), ctypes.c_int(self.rank),
            ctypes.c_int(self.world), ctypes.c_longlong(lo), ctypes.c_longlong(hi), ctypes.c_float(scale),
            *epoch, ctypes.c_int(self.max_ctas), _lib.ptr(_lib.status_word(self.tensor.device)),
            _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_allreduce")
        _lib.count(1)

    def _call(self, fn, lo: int, hi: int, scale: float, name: str, multicast: bool) -> None:
        epoch = self._next_epoch()
        rc = fn(
            _lib.ptr(self._peer_ptrs), _lib.ptr(self._pad_ptrs), ctypes.c_ulonglong(self.multicast_ptr if multicast else 0), ctypes.c_int(self.rank),
            ctypes.c_int(self.world), ctypes.c_longlong(lo), ctypes.c_longlong(hi), ctypes.c_float(scale), *epoch,
            ctypes.c_int(self.max_ctas), _lib.ptr(_lib.status_word(self.tensor.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, name)
        _lib.count(1)

    def all_reduce_bf16_(self, lo: int, hi: int) -> None:
        """In-place sum over ranks of ``tensor[lo:hi]`` of a bf16 buffer (bounds multiples of 8), fp32 accumulation."""
        assert self.tensor.dtype == torch.bfloat16
        epoch = self._next_epoch()
        rc = _lib.load().sb_allreduce_bf16(
            _lib.ptr(self._peer_ptrs), _lib.ptr(self._pad_ptrs), ctypes.c_ulonglong(self.multicast_ptr if self.use_multimem else 0),
            ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_longlong(lo), ctypes.c_longlong(hi), *epoch,
            ctypes.c_int(self.max_ctas), _lib.ptr(_lib.status_word(self.tensor.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_allreduce_bf16")
        _lib.count(1)

    def reduce_to_owner_(self, lo: int, hi: int, own_lo: int, own_hi: int, average: bool = True) -> None:
        """Sum (or mean) of ``tensor[lo:hi]`` across ranks, delivered only to owners: this rank ends up with the reduced
        ``tensor[own_lo:own_hi]`` in its own copy (the rest of ``[lo, hi)`` keeps its local values).  fp32 buffers only."""
        assert self.tensor.dtype == torch.float32
        epoch = self._next_epoch()
        rc = _lib.load().sb_reduce_to_owner(
            _lib.ptr(self._peer_ptrs), _lib.ptr(self._pad_ptrs), ctypes.c_ulonglong(self.multicast_ptr if self.use_multimem else 0),
            ctypes.c_int(self.rank), ctypes.c_int(self.world), ctypes.c_longlong(lo), ctypes.c_longlong(hi), ctypes.c_longlong(own_lo),
            ctypes.c_longlong(own_hi), ctypes.c_float(1.0 / self.world if average else 1.0), *epoch,
            ctypes.c_int(self.max_ctas), _lib.ptr(_lib.status_word(self.tensor.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_reduce_to_owner")
        _lib.count(1)

    def all_gather_slices_(self, lo: int, hi: int, average: bool = True) -> None:
        """Every rank broadcasts its 1/W slice of ``tensor[lo:hi]`` to all ranks (second half of an all-reduce whose
        reduce-scatter was done by the producing kernels adding into the owner's copy)."""
        self._call(_lib.load().sb_allgather_slices, lo, hi, 1.0 / self.world if average else 1.0, "sb_allgather_slices", self.use_multimem)

    def barrier(self) -> None:
        """Cross-rank barrier as a kernel on the current stream (bounded wait; a late peer sets the status word)."""
        epoch = self._next_epoch()
        rc = _lib.load().sb_rank_barrier(_lib.ptr(self._pad_ptrs), ctypes.c_int(self.rank), ctypes.c_int(self.world), *epoch,
                                         _lib.ptr(_lib.status_word(self.tensor.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "sb_rank_barrier")
        _lib.count(1)

    @property
    def peer_ptrs(self) -> torch.Tensor:
        return self._peer_ptrs

    def slice_vecs(self, lo: int, hi: int) -> int:
        """16-byte elements per owner slice of ``[lo, hi)`` (the split the reduction kernels use)."""
        vecs = (hi - lo) // 4
        return max(1, (vecs + self.world - 1) // self.world)
