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


def backward_supported(q: torch.Tensor) -> bool:
    return q.shape[-1] == 128


def backward(q, k, v, out, dout, lse, dq, dk, dv, *, causal: bool, key_mask=None, scale: float | None = None) -> None:
    """Gradients of ``forward`` written into ``dq, dk, dv`` (``[B, H, S, D]`` views with the token-major layout of the
    sources, e.g. views of one fused QKV gradient matrix).  ``out`` and ``dout`` are ``[B, S, H * D]``; head_dim 128."""
    b, h, s, d = q.shape
    assert d == 128, "the in-tree attention backward is written for head_dim 128"
    for t in (q, k, v, dq, dk, dv):
        assert _token_major(t), "operands must be token-major views (see _token_major)"
    assert q.stride(1) == k.stride(1) == v.stride(1) and dq.stride(1) == dk.stride(1) == dv.stride(1)
    out2 = out.reshape(b * s, h * d)
    dout2 = dout.reshape(b * s, h * d).contiguous()
    assert out2.is_contiguous() and out2.dtype == torch.bfloat16 and dout2.dtype == torch.bfloat16
    delta = torch.empty(b, h, s, dtype=torch.float32, device=q.device)
    dq32 = torch.empty(b * s, h * d, dtype=torch.float32, device=q.device)
    mask = key_mask.to(torch.uint8).contiguous() if key_mask is not None else None
    rc = _lib.load().sb_flash_bwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), c_int(q.stride(2)), c_int(k.stride(2)), c_int(v.stride(2)), c_int(0), c_int(0), c_int(0),
        c_int(q.stride(1)), _lib.ptr(out2), _lib.ptr(dout2), _lib.ptr(lse), _lib.ptr(mask), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
        c_int(dq.stride(2)), c_int(dk.stride(2)), c_int(dv.stride(2)), c_int(0), c_int(0), c_int(0), c_int(dq.stride(1)), _lib.ptr(delta),
        _lib.ptr(dq32), c_int(b), c_int(h), c_int(s), c_int(d), c_float(scale if scale is not None else 1.0 / math.sqrt(d)), c_int(int(causal)),
        c_int(_lib.sm_count(q.device)), _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_flash_bwd")
    _lib.count(3)


def qkv_views(qkv2d: torch.Tensor, b: int, s: int, h: int, d: int, layout: str):
    """``[B, H, S, D]`` views of q, k, v inside a fused projection output ``[B * S, 3 * H * D]``: ``interleaved`` = per head
    ``[q | k | v]`` (GPT-NeoX), ``blocked`` = ``[Q | K | V]`` (GPT-2, BERT)."""
    if layout == "interleaved":
        return tuple(t.transpose(1, 2) for t in qkv2d.view(b, s, h, 3 * d).split(d, dim=-1))
    if layout == "blocked":
        return tuple(t.view(b, s, h, d).transpose(1, 2) for t in qkv2d.split(h * d, dim=-1))
    raise ValueError(f"unknown QKV layout {layout!r}")


class _FusedQKVAttentionFn(torch.autograd.Function):
    """Attention straight on the fused QKV projection output: forward and backward read q, k, v in place and the backward
    writes dq, dk, dv into one gradient matrix of the same layout, so no split / cat / transpose copy exists on either pass."""

    @staticmethod
    def forward(ctx, qkv2d, b, s, h, d, layout, causal, key_mask):
        q, k, v = qkv_views(qkv2d, b, s, h, d, layout)
        out, lse = forward(q, k, v, causal=causal, key_mask=key_mask)
        ctx.save_for_backward(qkv2d, out, lse)
        ctx.meta = (b, s, h, d, layout, causal)
        ctx.key_mask = key_mask
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv2d, out, lse = ctx.saved_tensors
        b, s, h, d, layout, causal = ctx.meta
        dqkv = torch.empty_like(qkv2d)
        q, k, v = qkv_views(qkv2d, b, s, h, d, layout)
        dq, dk, dv = qkv_views(dqkv, b, s, h, d, layout)
        backward(q, k, v, out, dout, lse, dq, dk, dv, causal=causal, key_mask=ctx.key_mask)
        return dqkv, None, None, None, None, None, None, None


def fused_qkv_attention(qkv2d: torch.Tensor, b: int, s: int, h: int, d: int, *, layout: str, causal: bool, key_mask=None) -> torch.Tensor:
    """Context ``[B, S, H * D]`` from a fused QKV projection output ``[B * S, 3 * H * D]`` (bf16, CUDA, head_dim 128), with an
    in-tree backward.  See ``fused_supported``."""
    return _FusedQKVAttentionFn.apply(qkv2d, b, s, h, d, layout, causal, key_mask)


def fused_supported(qkv2d: torch.Tensor, d: int) -> bool:
    return qkv2d.is_cuda and qkv2d.dtype == torch.bfloat16 and qkv2d.dim() == 2 and qkv2d.is_contiguous() and d == 128 and _lib.available()


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
