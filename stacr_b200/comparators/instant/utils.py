"""Seeding and subspace-shape logging (parity: comparators/instant/utils.py)."""

from __future__ import annotations

import json
import os
import random

import numpy as np
import torch


def set_train_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def log_svd_shapes(iteration, U_dict: dict, output_file: str) -> None:
    """Append ``{iteration: {layer: {"shape": [...]}}}`` to a JSON file; values are tensors or ``(tensor, ...)`` tuples."""
    results = {}
    if os.path.exists(output_file) and os.path.getsize(output_file):
        with open(output_file) as fh:
            results = json.load(fh)
    entry = results.setdefault(str(iteration), {})
    for layer, value in U_dict.items():
        tensor = value[0] if isinstance(value, (tuple, list)) else value
        entry[layer] = {"shape": list(tensor.shape)}
    with open(output_file, "w") as fh:
        json.dump(results, fh, indent=2)
