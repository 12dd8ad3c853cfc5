"""Matrix <-> higher-order tensor reshapes used by the TT/Tucker comparators (parity: stacr/protocols/reshape.py)."""

from __future__ import annotations

import math

import torch


class Reshaper:
    @staticmethod
    def to_tensor(matrix_input: torch.Tensor, target_shape):
        shape = tuple(int(d) for d in target_shape)
        if math.prod(shape) != matrix_input.numel():
            raise ValueError(f"Cannot reshape {tuple(matrix_input.shape)} into {shape}")
        return matrix_input.reshape(shape)

    @staticmethod
    def to_matrix(tensor_input: torch.Tensor):
        return tensor_input.reshape(tensor_input.shape[0], -1) if tensor_input.dim() > 2 else tensor_input
