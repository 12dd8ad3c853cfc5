"""Seeding for protocol runs (parity: stacr/protocols/utils.py:1-30 of the reference project)."""

from __future__ import annotations

import os
import random

import numpy as np
import torch


def set_all_seeds(seed: int = 42, *, strict: bool = False) -> int:
    """Seed python, numpy and torch; ``strict`` also forces deterministic algorithms and disables TF32."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if strict:
        torch.use_deterministic_algorithms(True)
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if strict or torch.cuda.is_available():
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
    return seed
