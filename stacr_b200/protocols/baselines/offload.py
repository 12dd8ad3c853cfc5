"""Saved-tensor host-offload baseline with timing statistics.

Parity: stacr/protocols/baselines/offload.py:16-218 of the reference project (modes ``cpu`` and
``cpu_pinned``, ``min_bytes`` threshold, per-direction byte and time counters, RSS tracking).
"""

from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Any, Dict, Tuple

import torch


class SavedTensorOffloader:
    def __init__(self, mode: str = "cpu", min_bytes: int = 1_000_000):
        if mode not in ("cpu", "cpu_pinned"):
            raise ValueError("mode must be 'cpu' or 'cpu_pinned'")
        self.mode, self.min_bytes = mode, int(min_bytes)
        self.reset()

    def reset(self) -> None:
        self.pack_count = self.unpack_count = self.skipped = 0
        self.bytes_offloaded = self.bytes_restored = 0
        self.pack_seconds = self.unpack_seconds = 0.0

    def pack(self, tensor: torch.Tensor) -> Tuple[Any, torch.device, torch.dtype]:
        nbytes = tensor.numel() * tensor.element_size()
        if tensor.device.type == "cpu" or nbytes < self.min_bytes or tensor.layout != torch.strided:
            self.skipped += 1
            return tensor, tensor.device, tensor.dtype
        t0 = time.perf_counter()
        if self.mode == "cpu_pinned":
            host = torch.empty_like(tensor, device="cpu", pin_memory=True, memory_format=torch.preserve_format)
            host.copy_(tensor, non_blocking=True)
            torch.cuda.current_stream(tensor.device).synchronize()
        else:
            host = tensor.detach().cpu()
        self.pack_seconds += time.perf_counter() - t0
        self.pack_count += 1
        self.bytes_offloaded += nbytes
        return host, tensor.device, tensor.dtype

    def unpack(self, packed: Tuple[Any, torch.device, torch.dtype]) -> torch.Tensor:
        host, device, _ = packed
        if host.device == device:
            return host
        t0 = time.perf_counter()
        out = host.to(device, non_blocking=host.is_pinned())
        self.unpack_seconds += time.perf_counter() - t0
        self.unpack_count += 1
        self.bytes_restored += host.numel() * host.element_size()
        return out

    @contextmanager
    def context(self):
        with torch.autograd.graph.saved_tensors_hooks(self.pack, self.unpack):
            yield self

    def get_timing_stats(self) -> Dict[str, Any]:
        return {
            "mode": self.mode, "min_bytes": self.min_bytes, "pack_count": self.pack_count, "unpack_count": self.unpack_count,
            "skipped": self.skipped, "bytes_offloaded": self.bytes_offloaded, "bytes_restored": self.bytes_restored,
            "pack_seconds": self.pack_seconds, "unpack_seconds": self.unpack_seconds,
            "offload_GBps": self.bytes_offloaded / self.pack_seconds / 1e9 if self.pack_seconds else None,
            "restore_GBps": self.bytes_restored / self.unpack_seconds / 1e9 if self.unpack_seconds else None,
        }


class OffloadManager:
    """Owns an offloader and tracks host RSS around training steps."""

    def __init__(self, mode: str = "cpu", min_bytes: int = 1_000_000):
        self.offloader = SavedTensorOffloader(mode, min_bytes)
        self.peak_rss = 0

    def _get_rss(self) -> int:
        try:
            import psutil

            return int(psutil.Process().memory_info().rss)
        except Exception:
            return 0

    @contextmanager
    def training_step(self):
        with self.offloader.context():
            yield
        self.peak_rss = max(self.peak_rss, self._get_rss())

    def get_stats(self) -> Dict[str, Any]:
        return {**self.offloader.get_timing_stats(), "peak_rss_bytes": self.peak_rss}

    def reset(self) -> None:
        self.offloader.reset()
        self.peak_rss = 0
