"""Softmax attention on the in-tree tcgen05 kernels (``csrc/attention.cu``): no ``S x S`` tensor, no library kernel.

``flash_attention(q, k, v, causal=..., key_mask=...)`` takes ``[B, H, S, D]`` tensors and returns the context as
``[B, S, H * D]`` (the layout the output projection wants, so no transpose copy follows).  The inputs may be strided views
of a fused QKV projection output (``[B * S, 3 * H * D]``, interleaved per head or not): the kernels address them through
tensor maps and read them in place.  ``D`` is 64 or 128; other head sizes, other dtypes and CPU tensors go through
``torch``'s reference formula (``supported`` tells which).

The reference computes TP attention as eager scores + softmax (stacr/protocols/tp_gpt2.py:256-283 there) and otherwise
whatever the Hugging Face model does (SDPA).
"""

from __future__ import annotations

import math
from ctypes import c_float, c_int

import torch

from . import _lib


def _token_major(t: torch.Tensor) -> bool:
    """``t[b, h, s, :]`` lives at ``base + (b * S + s) * ld + h * head_stride`` with TMA-compatible alignment."""
    b, h, s, d = t.shape
    sb, sh, ss, sd = t.stride()
    return (sd == 1 and (b == 1 or sb == s * ss) and ss % 8 == 0 and sh % 8 == 0 and ss >= (h - 1) * sh + d and t.data_ptr() % 16 == 0)


def _as_token_major(t: torch.Tensor) -> torch.Tensor:
    return t if _token_major(t) else t.transpose(1, 2).contiguous().transpose(1, 2)


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == k.dtype == v.dtype == torch.bfloat16 and q.dim() == 4 and q.shape == k.shape == v.shape
            and q.shape[-1] in (64, 128) and _lib.available())


def forward(q, k, v, *, causal: bool, key_mask=None, scale: float | None = None, need_lse: bool = True):
    """Returns ``(out [B, S, H * D] bf16, lse [B, H, S] fp32 or None)``."""
    b, h, s, d = q.shape
    q, k, v = _as_token_major(q), _as_token_major(k), _as_token_major(v)
    if q.stride(1) != k.stride(1) or q.stride(1) != v.stride(1):
        # one head stride for the three operands: give each its own dense copy
        q, k, v = (t.transpose(1, 2).contiguous().transpose(1, 2) for t in (q, k, v))
    out = torch.empty(b, s, h * d, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, h, s, dtype=torch.float32, device=q.device) if need_lse else None
    mask = None
    if key_mask is not None:
        mask = key_mask.to(torch.uint8).contiguous()
    rc = _lib.load().sb_flash_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), c_int(q.stride(2)), c_int(k.stride(2)), c_int(v.stride(2)), c_int(0), c_int(0), c_int(0),
        c_int(q.stride(1)), _lib.ptr(out), c_int(h * d), _lib.ptr(lse) if lse is not None else None, _lib.ptr(mask) if mask is not None else None,
        c_int(b), c_int(h), c_int(s), c_int(d), c_float(scale if scale is not None else 1.0 / math.sqrt(d)), c_int(int(causal)),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_flash_fwd")
    _lib.count(1)
    return out, lse


def reference(q, k, v, *, causal: bool, key_mask=None, scale: float | None = None) -> torch.Tensor:
    """The plain formula in fp32 (oracle for the tests, and the path for unsupported inputs): ``[B, S, H * D]``."""
    b, h, s, d = q.shape
    scores = (q.float() @ k.float().transpose(-1, -2)) * (scale if scale is not None else 1.0 / math.sqrt(d))
    if causal:
        scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    if key_mask is not None:
        scores = scores.masked_fill(~key_mask.to(torch.bool)[:, None, None, :], float("-inf"))
    probs = torch.softmax(scores, dim=-1).nan_to_num(0.0)
    return (probs @ v.float()).transpose(1, 2).reshape(b, s, h * d)
