"""ctypes entry points for ``csrc/nn_kernels.cu`` (LayerNorm, GELU, cross-entropy, casts)."""

from __future__ import annotations

import ctypes

import torch

from . import _lib

c_int, c_ll, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _f32(t):
    return None if t is None else t.detach().float().contiguous()


def layernorm_fwd(x2d: torch.Tensor, weight, bias, eps: float):
    rows, n = x2d.shape
    y = torch.empty_like(x2d)
    mean = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    rc = _lib.load().sb_layernorm_fwd(_lib.ptr(x2d), _lib.ptr(_f32(weight)), _lib.ptr(_f32(bias)), c_int(rows), c_int(n), c_float(eps),
                                      _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_layernorm_fwd")
    _lib.count(1)
    return y, mean, rstd


def layernorm_bwd(dy2d, x2d, weight, mean, rstd):
    rows, n = x2d.shape
    dx = torch.empty_like(x2d)
    dwb = torch.zeros(2, n, dtype=torch.float32, device=x2d.device)
    rc = _lib.load().sb_layernorm_bwd(_lib.ptr(dy2d), _lib.ptr(x2d), _lib.ptr(_f32(weight)), _lib.ptr(mean), _lib.ptr(rstd), c_int(rows),
                                      c_int(n), _lib.ptr(dx), _lib.ptr(dwb[0]), _lib.ptr(dwb[1]), c_int(_lib.sm_count(x2d.device)),
                                      _lib.stream_ptr())
    _lib.check_rc(rc, "sb_layernorm_bwd")
    _lib.count(2)
    return dx, dwb[0], dwb[1]


def layernorm_fwd2(x2d: torch.Tensor, w1, b1, w2, b2, eps: float):
    """Two affine outputs of one normalisation of ``x2d`` (one read of the input, shared statistics)."""
    rows, n = x2d.shape
    y1, y2 = torch.empty_like(x2d), torch.empty_like(x2d)
    mean = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device)
    rc = _lib.load().sb_layernorm_fwd2(_lib.ptr(x2d), _lib.ptr(_f32(w1)), _lib.ptr(_f32(b1)), _lib.ptr(_f32(w2)), _lib.ptr(_f32(b2)), c_int(rows),
                                       c_int(n), c_float(eps), _lib.ptr(y1), _lib.ptr(y2), _lib.ptr(mean), _lib.ptr(rstd), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_layernorm_fwd2")
    _lib.count(1)
    return y1, y2, mean, rstd


def layernorm_bwd2(dy1, dy2, res, x2d, w1, w2, mean, rstd):
    """``dx = LNbwd(dy1; w1) + LNbwd(dy2; w2) + res`` in one pass, plus the four parameter gradients (fp32)."""
    rows, n = x2d.shape
    dx = torch.empty_like(x2d)
    grads = torch.zeros(4, n, dtype=torch.float32, device=x2d.device)
    rc = _lib.load().sb_layernorm_bwd2(_lib.ptr(dy1), _lib.ptr(dy2), _lib.ptr(res), _lib.ptr(x2d), _lib.ptr(_f32(w1)), _lib.ptr(_f32(w2)),
                                       _lib.ptr(mean), _lib.ptr(rstd), c_int(rows), c_int(n), _lib.ptr(dx), _lib.ptr(grads[0]), _lib.ptr(grads[1]),
                                       _lib.ptr(grads[2]), _lib.ptr(grads[3]), c_int(_lib.sm_count(x2d.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_layernorm_bwd2")
    _lib.count(3)
    return dx, grads[0], grads[1], grads[2], grads[3]


def add3(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(a)
    rc = _lib.load().sb_add3(_lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.ptr(out), c_ll(a.numel()), c_int(_lib.sm_count(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_add3")
    _lib.count(1)
    return out


def gelu_fwd(x: torch.Tensor, tanh_form: bool) -> torch.Tensor:
    y = torch.empty_like(x)
    rc = _lib.load().sb_gelu_fwd(_lib.ptr(x), _lib.ptr(y), c_ll(x.numel()), c_int(int(tanh_form)), c_int(_lib.sm_count(x.device)),
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "sb_gelu_fwd")
    _lib.count(1)
    return y


def gelu_bwd(dy: torch.Tensor, x: torch.Tensor, tanh_form: bool) -> torch.Tensor:
    dx = torch.empty_like(x)
    rc = _lib.load().sb_gelu_bwd(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(dx), c_ll(x.numel()), c_int(int(tanh_form)),
                                 c_int(_lib.sm_count(x.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_gelu_bwd")
    _lib.count(1)
    return dx


def gelu_bwd_colsum(dy: torch.Tensor, x: torch.Tensor, tanh_form: bool):
    """``(dx, column sums of dx)`` for contiguous bf16 ``[..., n]`` with ``n % 8 == 0``; the sums are fp32 ``[n]``."""
    n = x.shape[-1]
    rows = x.numel() // n
    dx = torch.empty_like(x)
    sums = torch.zeros(n, dtype=torch.float32, device=x.device)
    rc = _lib.load().sb_gelu_bwd_colsum(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(dx), c_int(rows), c_int(n), c_int(int(tanh_form)), _lib.ptr(sums),
                                        c_int(_lib.sm_count(x.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_gelu_bwd_colsum")
    _lib.count(1)
    return dx, sums


def cross_entropy_fwd(logits: torch.Tensor, target: torch.Tensor):
    """Mean loss over valid rows; returns ``(loss, target_int64, row_lse, inv_valid)`` for :func:`cross_entropy_bwd`."""
    rows, v = logits.shape
    target = target.to(torch.int64)
    inv_valid = 1.0 / (target != -100).sum().clamp_min(1).float()
    row_loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    row_lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = _lib.load().sb_cross_entropy(_lib.ptr(logits), _lib.ptr(target), c_int(rows), c_int(v), _lib.ptr(inv_valid), _lib.ptr(None),
                                      _lib.ptr(row_loss), _lib.ptr(row_lse), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_cross_entropy")
    _lib.count(1)
    return row_loss.sum() * inv_valid, target, row_lse, inv_valid


def cross_entropy_bwd(logits: torch.Tensor, target: torch.Tensor, row_lse: torch.Tensor, inv_valid: torch.Tensor, dloss: torch.Tensor) -> torch.Tensor:
    """``d loss / d logits`` scaled by the upstream scalar ``dloss`` (a device tensor: no host read)."""
    rows, v = logits.shape
    dlogits = torch.empty_like(logits)
    scale = dloss.detach().float().reshape(1)
    rc = _lib.load().sb_cross_entropy_bwd(_lib.ptr(logits), _lib.ptr(target), c_int(rows), c_int(v), _lib.ptr(row_lse), _lib.ptr(inv_valid),
                                          _lib.ptr(scale), _lib.ptr(dlogits), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_cross_entropy_bwd")
    _lib.count(1)
    return dlogits


def cast_bf16(src: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16 copy (``numel % 4 == 0``)."""
    dst = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    rc = _lib.load().sb_cast_f32_bf16(_lib.ptr(src), _lib.ptr(dst), c_ll(src.numel()), c_int(_lib.sm_count(src.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_cast_f32_bf16")
    _lib.count(1)
    return dst


def rotary_qk_(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq: int, heads: int, head_dim: int, rot: int, sign: float) -> None:
    """In-place rotary embedding of the q and k parts of contiguous bf16 ``qkv`` ``[tokens, heads, 3*head_dim]``."""
    tokens = qkv.numel() // (heads * 3 * head_dim)
    rc = _lib.load().sb_rotary_qk(_lib.ptr(qkv), _lib.ptr(cos), _lib.ptr(sin), c_ll(tokens), c_int(seq), c_int(heads), c_int(head_dim),
                                  c_int(rot), c_float(sign), c_int(_lib.sm_count(qkv.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_rotary_qk")
    _lib.count(1)


def embedding_fwd(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """bf16 rows ``table[ids]`` from a bf16 or fp32 table ``[vocab, width]`` (``width % 8 == 0``); ids are checked on the device."""
    vocab, width = table.shape
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty(flat.numel(), width, dtype=torch.bfloat16, device=table.device)
    bad = torch.zeros(1, dtype=torch.int32, device=table.device)
    rc = _lib.load().sb_embedding_fwd(_lib.ptr(table), c_int(int(table.dtype == torch.bfloat16)), _lib.ptr(flat), c_ll(flat.numel()), c_int(width),
                                      c_int(vocab), _lib.ptr(out), _lib.ptr(bad), c_int(_lib.sm_count(table.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_embedding_fwd")
    _lib.count(1)
    return out.reshape(*ids.shape, width)


def embedding_bwd(dy: torch.Tensor, ids: torch.Tensor, vocab: int, padding_idx: int | None, out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``[vocab, width]`` gradient of the table: rows of ``dy`` (bf16) summed by id.  ``out`` (contiguous fp32) is cleared and filled."""
    width = dy.shape[-1]
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    d2 = dy.reshape(-1, width).contiguous()
    if out is None:
        out = torch.zeros(vocab, width, dtype=torch.float32, device=dy.device)
    else:
        out.zero_()
    rc = _lib.load().sb_embedding_bwd(_lib.ptr(d2), _lib.ptr(flat), c_ll(flat.numel()), c_int(width), c_int(vocab),
                                      c_ll(-1 if padding_idx is None else padding_idx), _lib.ptr(out), c_int(_lib.sm_count(dy.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "sb_embedding_bwd")
    _lib.count(1)
    return out
