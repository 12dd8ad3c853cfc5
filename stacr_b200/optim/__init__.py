"""Optimizers with native multi-tensor update kernels."""

from .adamw import AdamW, AdamW8bit

__all__ = ["AdamW", "AdamW8bit"]
