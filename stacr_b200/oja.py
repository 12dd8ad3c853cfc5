"""Orthonormal-basis maintenance: QR re-orthonormalisation and the Oja subspace tracker.

Parity target: stacr/oja.py:8-106 of the reference project.  The tracker fits the
*uncentred* activations on purpose (the reconstruction ``C Q^T`` never adds a mean back).
On CUDA the update of the compressed layers runs through the fused kernels in
``stacr_b200.ops.basis``; this module is the framework-level, device-agnostic form.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


def orthonormalize(matrix: torch.Tensor) -> torch.Tensor:
    """Orthonormal basis of the column span, computed in fp32 and returned in the input dtype."""
    q = torch.linalg.qr(matrix.float(), mode="reduced").Q
    return q.to(matrix.dtype)


def oja_step(basis: torch.Tensor, x: torch.Tensor, lr: float) -> torch.Tensor:
    """One Oja step ``Q <- orth(Q + lr (X^T Y / n - Q (Y^T Y) / n))`` with ``Y = X Q`` (fp32)."""
    q, xf = basis.float(), x.float()
    n = max(1, xf.shape[0])
    y = xf @ q
    delta = (xf.t() @ y - q @ (y.t() @ y)) / n
    return orthonormalize(q + float(lr) * delta)


def top_right_singular_basis(x: torch.Tensor, rank: int) -> torch.Tensor:
    """Top-``rank`` right singular vectors of ``x`` (rows >= rank), orthonormalised, fp32."""
    vh = torch.linalg.svd(x.float(), full_matrices=False).Vh
    return orthonormalize(vh[:rank].t().contiguous())


def seeded_random_basis(features: int, rank: int, device, seed: int = 0) -> torch.Tensor:
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    return orthonormalize(torch.randn(features, rank, generator=gen, dtype=torch.float32).to(device))


@dataclass
class OjaBasis:
    """Persistent per-feature-size basis updated from streamed activations.

    Every update *rebinds* ``basis`` to a new tensor, so a tensor handed out by
    :meth:`shared` stays valid for whoever saved it.
    """

    features: int
    rank: int
    dtype: torch.dtype = torch.float32
    device: torch.device | str = "cpu"
    initialized: bool = False
    basis: torch.Tensor = field(init=False, repr=False)

    def __post_init__(self) -> None:
        self.rank = max(1, min(int(self.rank), int(self.features)))
        self._cast_cache: dict[torch.dtype, torch.Tensor] = {}
        self.reset_random(seed=0)
        self.initialized = False

    def _set(self, fp32_basis: torch.Tensor) -> None:
        self.basis = fp32_basis.to(device=self.device, dtype=self.dtype)
        self._cast_cache = {}

    def reset_random(self, seed: int = 0) -> None:
        self._set(seeded_random_basis(self.features, self.rank, self.device, seed))
        self.initialized = True

    def initialize_from_batch(self, activations: torch.Tensor, centre: bool = False) -> None:
        x = activations.detach().reshape(-1, activations.shape[-1]).float()
        if centre:
            x = x - x.mean(0, keepdim=True)
        if x.shape[0] < self.rank:
            self.reset_random(seed=0)
            return
        self._set(top_right_singular_basis(x, self.rank))
        self.initialized = True

    @torch.no_grad()
    def update(self, activations: torch.Tensor, lr: float = 0.01) -> None:
        if not self.initialized:
            self.initialize_from_batch(activations)
            return
        x = activations.detach().reshape(-1, activations.shape[-1]).to(self.basis.device)
        if x.numel():
            self._set(oja_step(self.basis, x, lr))

    def snapshot(self, dtype: torch.dtype | None = None) -> torch.Tensor:
        out = self.basis.detach()
        return (out if dtype is None else out.to(dtype)).clone()

    def shared(self, dtype: torch.dtype | None = None) -> torch.Tensor:
        """Current basis version in ``dtype`` (cached cast), shared by all packs of this version."""
        want = self.basis.dtype if dtype is None else dtype
        hit = self._cast_cache.get(want)
        if hit is None:
            hit = self.basis.detach() if want == self.basis.dtype else self.basis.detach().to(want)
            self._cast_cache[want] = hit
        return hit
