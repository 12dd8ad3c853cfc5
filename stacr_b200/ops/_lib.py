"""ctypes binding to the in-tree sm_100a kernel library.

The library exposes a C ABI taking raw device pointers and a stream handle; the wrappers in
this package pass ``tensor.data_ptr()`` and ``torch.cuda.current_stream().cuda_stream``.
On a machine with a GPU a missing library is an error (no silent fallback to framework
ops); on a CPU-only machine the pure-PyTorch oracle paths are used and ``available()`` is
False.
"""

from __future__ import annotations

import ctypes
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
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists():
                from .build import ensure_built

                ensure_built()
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
