"""bf16 tensor-core GEMM (tcgen05/TMEM/TMA kernel in ``csrc/gemm_tc.cu``)."""

from __future__ import annotations

import ctypes

import torch

from . import _lib


import os

_TWO_CTA_DEFAULT = os.environ.get("STACR_GEMM_2CTA", "1") == "1"


_TYPED = None


def _typed_lib():
    """The kernel library with argument types declared for the two GEMM entry points: plain Python ints and floats are
    converted by ctypes itself, which is several microseconds cheaper per launch than building c_int / c_void_p objects."""
    global _TYPED
    if _TYPED is None:
        lib = _lib.load()
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.sb_gemm_bf16.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp, vp]
        lib.sb_gemm_bf16.restype = ci
        lib.sb_gemm_bf16_2cta.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp, vp]
        lib.sb_gemm_bf16_2cta.restype = ci
        _TYPED = lib
    return _TYPED


def _pick_bn(m: int, n: int, b_mn: bool, sms: int) -> int:
    if n <= 16 and not b_mn:
        return 16
    if n <= 32 and not b_mn:
        return 32
    if n <= 64:
        return 64
    num_m = (m + 127) // 128
    best, best_score = 128, -1.0
    for bn, weight in ((256, 1.0), (128, 0.85)):
        if bn == 256 and n <= 128:
            continue
        tiles = num_m * ((n + bn - 1) // bn)
        waves = (tiles + sms - 1) // sms
        score = weight * tiles / (waves * sms) * (n / (((n + bn - 1) // bn) * bn))
        if score > best_score:
            best, best_score = bn, score
    return best


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    splits: int = 1,
    bn: int | None = None,
    alpha: float = 1.0,
    two_cta: bool | None = None,
) -> torch.Tensor:
    """``out[M,N] = alpha * A @ B^T (+ bias)`` with bf16 operands and fp32 accumulation.

    ``a`` is ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b`` is ``[N,K]``
    (``b_mn=False``) or ``[K,N]`` (``b_mn=True``).  Rows of both must be contiguous.
    With ``splits > 1`` (or an explicit fp32 ``out`` passed with ``splits=0`` meaning
    "accumulate into out") partial tiles are reduced with fp32 atomics into ``out``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "operands must be bf16"
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        k, m = a.shape
    else:
        m, k = a.shape
    if b_mn:
        kb, n = b.shape
    else:
        n, kb = b.shape
    assert k == kb, f"reduction mismatch {k} vs {kb}"
    accumulate_into = out is not None and splits == 0
    if accumulate_into:
        splits = 1
    atomic = splits > 1 or accumulate_into
    if out is None:
        dtype = torch.float32 if atomic else out_dtype
        out = (torch.zeros if atomic else torch.empty)((m, n), dtype=dtype, device=a.device)
    else:
        assert out.shape == (m, n) and out.stride(1) == 1
    if atomic:
        assert out.dtype == torch.float32
        mode = 2
    else:
        mode = {torch.bfloat16: 0, torch.float32: 1}[out.dtype]
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n and bias.is_contiguous()
    sms = _lib.sm_count(a.device)
    if bn is None:
        bn = _pick_bn(m, n, b_mn, sms)
    lib = _typed_lib()
    if two_cta is None:
        two_cta = _TWO_CTA_DEFAULT and bn == 256 and m >= 512 and n >= 512
    bias_ptr = None if bias is None else bias.data_ptr()
    status = _lib.status_word(a.device).data_ptr()
    stream = _lib.stream_ptr()
    if two_cta and not atomic:
        # CTA pairs on 256 x 256 tiles (tcgen05.mma.cta_group::2): each CTA stages half of the B tile
        rc = lib.sb_gemm_bf16_2cta(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_ptr, m, n, k, a.stride(0), b.stride(0), out.stride(0),
                                   int(a_mn), int(b_mn), mode, alpha, sms, status, stream)
        _lib.check_rc(rc, "sb_gemm_bf16_2cta")
        _lib.count(1)
        return out
    rc = lib.sb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_ptr, m, n, k, a.stride(0), b.stride(0), out.stride(0),
                          int(a_mn), int(b_mn), mode, max(1, splits), bn, alpha, sms, status, stream)
    _lib.check_rc(rc, "sb_gemm_bf16")
    _lib.count(1)
    return out
