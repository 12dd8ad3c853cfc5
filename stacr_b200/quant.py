"""Symmetric per-tensor quantisation of the sparse residual values.

Behavioural parity with the reference's value codec (stacr/quant.py:8-65 there): one fp32
scale per tensor, ``qmax`` 127 (int8) or 7 (int4), rounding to nearest, clamp to the full
two's-complement range, two nibbles per byte with the even element in the low nibble.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

_QMAX = {4: 7.0, 8: 127.0}


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """Pack signed nibbles (-8..7), two per byte, even index in the low half."""
    v = values.reshape(-1).to(torch.int8)
    if v.numel() & 1:
        v = torch.nn.functional.pad(v, (0, 1))
    pairs = v.view(-1, 2).to(torch.uint8) & 0x0F
    return (pairs[:, 0] | (pairs[:, 1] << 4)).contiguous()


def unpack_int4(packed: torch.Tensor, length: int) -> torch.Tensor:
    """Inverse of :func:`pack_int4`; returns ``length`` int8 values."""
    b = packed.reshape(-1).to(torch.uint8)
    nib = torch.stack((b & 0x0F, (b >> 4) & 0x0F), dim=1).reshape(-1).to(torch.int8)
    nib = nib - ((nib > 7).to(torch.int8) << 4)  # sign-extend the nibble
    return nib[:length]


@dataclass
class QuantizedValues:
    """A 1-D value vector held as integers plus one scale (or raw when ``bits == 0``)."""

    data: torch.Tensor
    scale: torch.Tensor
    bits: int
    length: int

    def dequantize(self, dtype: torch.dtype) -> torch.Tensor:
        ints = unpack_int4(self.data, self.length) if self.bits == 4 else self.data
        return ints.to(dtype) * self.scale.to(dtype)

    def stored_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.data, self.scale))


def quantize_values(values: torch.Tensor, bits: int) -> QuantizedValues:
    """Quantise ``values`` to ``bits`` in {0, 4, 8}; ``0`` keeps the tensor untouched."""
    if bits not in (0, 4, 8):
        raise ValueError("residual_bits must be 0, 4, or 8")
    flat = values.reshape(-1)
    n = int(flat.numel())
    if bits == 0 or n == 0:
        unit = torch.ones((), dtype=torch.float32, device=flat.device)
        return QuantizedValues(flat, unit, 0, n)
    qmax = _QMAX[bits]
    f = flat.float()
    scale = (f.abs().amax() / qmax).clamp_min(torch.finfo(torch.float32).tiny)
    q = torch.round(f / scale).clamp_(-qmax - 1.0, qmax).to(torch.int8)
    return QuantizedValues(pack_int4(q) if bits == 4 else q, scale.reshape(()).float(), bits, n)
