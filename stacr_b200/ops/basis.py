"""Basis initialisation and tracking on the kernel path.

* ``oja_step_kernels``: ``Y = X Q`` (tensor-core projection), ``G = X^T Y`` (skinny MN-major
  tensor-core product), then the fused Oja + CholeskyQR2 kernel.  Three passes over ``X`` become
  two, with no fp32 copy of ``X`` (the reference copies ``X`` to fp32 and issues four GEMMs and a
  QR: stacr/layers.py:350-353 there).
* ``range_finder_basis``: randomized subspace iteration for the first basis instead of a full
  SVD of the ``rows x features`` activation (stacr/layers.py:331-335 there), followed by a
  Rayleigh-Ritz rotation so the columns are ordered by captured energy.
"""

from __future__ import annotations

import torch

from . import stacr_ops


@torch.no_grad()
def oja_step_kernels(basis: torch.Tensor, x: torch.Tensor, lr: float) -> torch.Tensor:
    """One Oja update of ``basis`` ``[N, r]`` from bf16 ``x`` ``[rows, N]``; returns the fp32 basis.

    The bf16 views the forward needs are attached to the returned tensor so they are not rebuilt.
    """
    rows, _ = x.shape
    r = basis.shape[1]
    x = x.contiguous()
    views = getattr(basis, "_sb_views", None)
    if views is None:
        qb = basis.detach().to(torch.bfloat16).contiguous()
        views = (qb, stacr_ops.pad_basis_transpose(qb))
    y = stacr_ops.project(x, views[1])  # [rows, rpad] fp32
    g = stacr_ops.at_b(x, stacr_ops.transpose_pad(y[:, :r]))  # [N, rpad] fp32
    new_q, qb, qt = stacr_ops.oja_update(basis.detach().float(), g, y, rows, lr)
    new_q._sb_views = (qb, qt)
    return new_q


@torch.no_grad()
def range_finder_basis(x: torch.Tensor, rank: int, iters: int = 4, oversample: int = 8) -> torch.Tensor:
    """Approximate top-``rank`` right singular subspace of bf16 ``x`` by subspace iteration.

    Every step is an in-tree kernel: the two skinny products on the tensor cores, the orthonormalisation of the
    ``[features, width]`` iterate by Gram-Schmidt with re-orthogonalisation, the ``width x width`` Gram matrix of the projected
    rows in fp64, and its eigen-decomposition by Jacobi rotations (no library QR or eigensolver is called).
    """
    rows, n = x.shape
    x = x.contiguous()
    width = min(32, rank + oversample, n)
    gen = torch.Generator(device="cpu").manual_seed(0)
    q = stacr_ops.orthonormalize_columns_(torch.randn(n, width, generator=gen).to(x.device).contiguous())
    for _ in range(iters):
        qt = stacr_ops.pad_basis_transpose(q.to(torch.bfloat16).contiguous())
        y = stacr_ops.project(x, qt)[:, :width]
        g = stacr_ops.at_b(x, stacr_ops.transpose_pad(y))[:, :width]
        q = stacr_ops.orthonormalize_columns_(g.contiguous())
    qt = stacr_ops.pad_basis_transpose(q.to(torch.bfloat16).contiguous())
    y = stacr_ops.project(x, qt)[:, :width].contiguous()
    _, evecs = stacr_ops.small_eigh(stacr_ops.small_gram(y))
    # rotate the iterate so that its columns are ordered by captured energy, keep the leading ones; the product of a matrix with
    # orthonormal columns and an orthogonal one has orthonormal columns, one Gram-Schmidt pass removes the rounding
    rotated = torch.zeros(n, rank, dtype=torch.float32, device=x.device)
    lead = evecs[:, :rank].float()
    for j in range(width):           # width <= 32 rank-one accumulations of an [n, rank] matrix: element-wise kernels only
        rotated.addcmul_(q[:, j:j + 1], lead[j:j + 1, :])
    return stacr_ops.orthonormalize_columns_(rotated.contiguous())
