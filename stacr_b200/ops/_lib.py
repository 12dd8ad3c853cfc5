"""ctypes binding to the in-tree sm_100a kernel library.

The library exposes a C ABI taking raw device pointers and a stream handle; the wrappers in
this package pass ``tensor.data_ptr()`` and ``torch.cuda.current_stream().cuda_stream``.
On a machine with a GPU a missing library is an error (no silent fallback to framework
ops); on a CPU-only machine the pure-PyTorch oracle paths are used and ``available()`` is
False.
"""

from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libstacr_b200.so"
_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_status: dict[int, torch.Tensor] = {}
_sms: dict[int, int] = {}
_launches = 0

STATUS_TEXT = {
    0: "ok",
    11: "timeout waiting for a free shared-memory stage (producer)",
    12: "timeout waiting for a TMA tile to land (MMA issuer)",
    13: "timeout waiting for the epilogue to drain the accumulator",
    14: "timeout waiting for the accumulator to be produced (epilogue)",
    21: "timeout waiting for a peer rank's flag",
    31: "bad argument detected on the device",
}


class KernelError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """The kernel library, built first when it is missing or older than its sources.

    The build runs under a file lock and the link replaces the library atomically, so ranks started together by a launcher
    build once and never map a half-written file (see ``build.ensure_built``).
    """
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            from .build import ensure_built

            try:
                ensure_built()
            except OSError:
                if not _LIB_PATH.exists():
                    raise
            if not _LIB_PATH.exists():
                raise KernelError(
                    f"{_LIB_PATH} is missing: run `python -m stacr_b200.ops.build` (needs nvcc)"
                )
            _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


def available() -> bool:
    """True when a CUDA device is present (the kernel path is then mandatory)."""
    return torch.cuda.is_available()


def use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle (called once per kernel launch: kept cheap)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 word kernels write a non-zero code to when a bounded wait gives up."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    word = _status.get(idx)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = word
    return word


def check_status(device=None, *, reset: bool = True) -> None:
    """Synchronising read of the status word; raises KernelError on a recorded failure."""
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        if reset:
            word.zero_()
        raise KernelError(f"kernel status {code}: {STATUS_TEXT.get(code, 'unknown')}")


class _StatusPoller:
    """Asynchronous reader of one device's status word.

    ``poll`` queues a 4-byte copy of the word into pinned memory behind everything already on the current stream and
    inspects the copy queued by the previous call, so a training loop can look at the word every step without making the
    host wait for the GPU: a timeout recorded in step k raises at the end of step k + 1.
    """

    def __init__(self, device_index: int):
        self.index = device_index
        self.host = torch.zeros(2, dtype=torch.int32).pin_memory()
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.count = 0

    def poll(self, *, wait: bool = False) -> None:
        word = status_word(self.index)
        slot = self.count & 1
        prev = slot ^ 1
        if self.count:
            if wait:
                self.events[prev].synchronize()
            if self.events[prev].query():
                code = int(self.host[prev])
                if code != 0:
                    self.host[prev] = 0
                    word.zero_()
                    raise KernelError(f"kernel status {code}: {STATUS_TEXT.get(code, 'unknown')}")
        self.host[slot:slot + 1].copy_(word, non_blocking=True)
        self.events[slot].record()
        self.count += 1


_pollers: dict[int, _StatusPoller] = {}


def poll_status(device=None, *, strict: bool | None = None) -> None:
    """Non-blocking status check for training loops: raises ``KernelError`` for a failure recorded up to the previous call.

    With ``strict`` (or ``STACR_STRICT_STATUS=1``) the word is read synchronously instead, which costs a device
    synchronisation per call but reports a failure before anything consumes the step's results.
    """
    if not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        return
    if strict is None:
        strict = os.environ.get("STACR_STRICT_STATUS", "0") == "1"
    if strict:
        check_status(device)
        return
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    poller = _pollers.get(idx)
    if poller is None:
        poller = _pollers[idx] = _StatusPoller(idx)
    poller.poll()


_reserved_sms = 0


def reserve_sms(n: int) -> None:
    """Leave ``n`` SMs to kernels that run next to the compute stream (collectives overlapped with backward).

    The persistent GEMMs launch one CTA per SM and split their tiles statically among them; a CTA that finds its SM
    taken starts late and delays the whole kernel, so while a communication kernel is resident the GEMMs are launched
    with that many CTAs fewer.
    """
    global _reserved_sms
    _reserved_sms = max(0, int(n))


def sm_count(device=None) -> int:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx not in _sms:
        _sms[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return max(1, _sms[idx] - _reserved_sms)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def count(n: int = 1) -> None:
    """Record ``n`` launches of this library's kernels (read back with :func:`launch_count`)."""
    global _launches
    _launches += n


def launch_count() -> int:
    return _launches
