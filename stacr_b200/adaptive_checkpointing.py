"""Record/replay of per-layer compression state across activation-checkpoint recomputation.

A checkpointed block runs its forward twice.  The second run must see exactly the basis and
residual budget of the first, or the recomputed saved tensors (and so the weight gradient)
would differ from the direct run.  During the first forward every compressed layer appends
``(layer id, state)`` to a per-checkpoint list; during recomputation the list is replayed in
order.  Behavioural parity: stacr/adaptive_checkpointing.py:7-71 of the reference project.
"""

from __future__ import annotations

import threading
from contextlib import contextmanager


class RecomputationGuard:
    """Thread-local recorder/replayer.  One global instance serves every layer."""

    def __init__(self) -> None:
        self._tls = threading.local()

    # -- state accessors -------------------------------------------------------------
    @property
    def is_recomputing(self) -> bool:
        return bool(getattr(self._tls, "recomputing", False))

    def _sink(self):
        return getattr(self._tls, "sink", None)

    def _source(self):
        return getattr(self._tls, "source", None)

    # -- contexts ---------------------------------------------------------------------
    @contextmanager
    def forward_context(self, records: list):
        outer = self._sink()
        self._tls.sink = records
        try:
            yield
        finally:
            self._tls.sink = outer

    @contextmanager
    def recomputation_context(self, records=None):
        outer_flag, outer_source = self.is_recomputing, self._source()
        self._tls.recomputing = True
        self._tls.source = iter(records) if records is not None else None
        try:
            yield
        finally:
            self._tls.recomputing, self._tls.source = outer_flag, outer_source

    # -- layer hooks ------------------------------------------------------------------
    def record_layer(self, layer, state) -> None:
        sink = self._sink()
        if sink is not None and not self.is_recomputing:
            sink.append((id(layer), state))

    def replay_layer(self, layer):
        source = self._source()
        if source is None:
            return None
        entry = next(source, None)
        if entry is None:
            # nothing was recorded for this layer (the first forward ran without autograd, as a compressed
            # checkpoint boundary does): the replay is the layer's first training forward of the step
            return None
        ident, state = entry
        if ident != id(layer):
            raise RuntimeError("STAC-R layer order changed during checkpoint replay")
        return state


_GUARD = RecomputationGuard()


def get_global_recomputation_guard() -> RecomputationGuard:
    return _GUARD


def checkpoint_contexts():
    """``context_fn`` for ``torch.utils.checkpoint.checkpoint(use_reentrant=False)``."""
    log: list = []
    return _GUARD.forward_context(log), _GUARD.recomputation_context(log)


def checkpoint(function, *args, **kwargs):
    """Non-reentrant activation checkpoint that replays compression state on recomputation."""
    from torch.utils.checkpoint import checkpoint as _torch_checkpoint

    if kwargs.pop("use_reentrant", False):
        raise ValueError("Adaptive checkpointing requires use_reentrant=False")
    kwargs.setdefault("context_fn", checkpoint_contexts)
    return _torch_checkpoint(function, *args, use_reentrant=False, **kwargs)
