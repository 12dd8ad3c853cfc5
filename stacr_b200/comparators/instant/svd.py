"""Energy-thresholded eigenbasis of a token Gram matrix (parity: comparators/instant/svd.py)."""

from __future__ import annotations

import torch


def energy_basis(gram: torch.Tensor, var: float = 0.95, oversample: int = 7) -> torch.Tensor:
    """Columns spanning the leading singular directions of ``gram`` that hold ``var`` of its squared spectrum.

    The count is the number of cumulative-energy entries not above the threshold, plus ``oversample`` extra
    directions, plus one, capped at the matrix size.  The basis is divided by the square root of the retained
    energy fraction so that projecting and expanding keeps the expected squared norm.
    """
    u, s, _ = torch.linalg.svd(gram.float(), full_matrices=False)
    energy = s.square()
    total = energy.sum().clamp_min(1e-30)
    cum = energy.cumsum(0)
    keep = int((cum <= var * total).sum()) + int(oversample)
    width = u.shape[1]
    if keep + 1 < width:
        cols, kept = keep + 1, cum[keep + 1]
    else:
        cols, kept = min(max(keep, 1), width), total
    return u[:, :cols] / torch.sqrt(kept / total)


def SVD_expected_value(input: torch.Tensor, var: float = 0.95, p: int = 7) -> torch.Tensor:
    """Name used by the INSTANT scripts for :func:`energy_basis`."""
    return energy_basis(input, var=var, oversample=p)
from .utils import log_svd_shapes  # noqa: E402,F401  (also importable from here, as in the upstream layout)
