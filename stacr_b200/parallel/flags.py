"""Stream-ordered flag words: set, and wait with a time limit.

``wait(flag, expected, limit_s)`` enqueues a one-thread kernel that polls ``flag`` (acquire loads at system scope)
until it reaches ``expected`` or ``limit_s`` seconds pass; on expiry the kernel records a timeout in the device's
status word and returns, so the CUDA context stays usable and ``ops._lib.check_status()`` raises on the host.
This is the building block the in-kernel barriers use, exposed so that host code can bound a wait on a peer's
progress the same way (and so that the timeout path can be exercised without any peer at all).
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import _lib


def new_flag(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def set_(flag: torch.Tensor, value: int) -> None:
    rc = _lib.load().sb_flag_set(_lib.ptr(flag), ctypes.c_int(int(value)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_flag_set")
    _lib.count(1)


def wait(flag: torch.Tensor, expected: int, limit_s: float = 1.0, observed: torch.Tensor | None = None) -> None:
    rc = _lib.load().sb_flag_wait(_lib.ptr(flag), ctypes.c_int(int(expected)), ctypes.c_ulonglong(int(limit_s * 1e9)),
                                  _lib.ptr(_lib.status_word(flag.device)), _lib.ptr(observed), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_flag_wait")
    _lib.count(1)
