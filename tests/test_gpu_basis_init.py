"""The small dense algebra behind the basis initialisation against fp64 library results."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,w", [(8192, 16), (2048, 32), (100, 7), (33, 32)])
def test_gram_schmidt_kernel_orthonormalises_nearly_collinear_columns(n, w):
    from stacr_b200.ops import stacr_ops

    g = torch.Generator(device="cuda").manual_seed(n + w)
    base = torch.randn(n, 1, device="cuda", generator=g)
    a = (base * 100.0 + 1e-2 * torch.randn(n, w, device="cuda", generator=g)).contiguous()     # condition number ~1e4 and worse
    span = torch.linalg.qr(a.double()).Q
    q = stacr_ops.orthonormalize_columns_(a.clone())
    eye = torch.eye(w, device="cuda", dtype=torch.float64)
    assert float((q.double().t() @ q.double() - eye).abs().max()) < 1e-4
    # same column space: the projection of q onto the library's orthonormal basis loses nothing
    assert float((span @ (span.t() @ q.double()) - q.double()).abs().max()) < 1e-3


def test_gram_schmidt_kernel_replaces_a_vanishing_column():
    from stacr_b200.ops import stacr_ops

    a = torch.randn(512, 4, device="cuda")
    a[:, 2] = a[:, 0] * 3.0                     # exactly dependent
    q = stacr_ops.orthonormalize_columns_(a.contiguous())
    assert float((q.t() @ q - torch.eye(4, device="cuda")).abs().max()) < 1e-4


@pytest.mark.parametrize("w", [1, 5, 16, 32])
def test_jacobi_eigensolver_and_small_gram_match_fp64_library(w):
    from stacr_b200.ops import stacr_ops

    g = torch.Generator(device="cuda").manual_seed(w)
    y = (torch.randn(3000, w, device="cuda", generator=g) * torch.linspace(5.0, 0.1, w, device="cuda")).contiguous()
    gram = stacr_ops.small_gram(y)
    want = y.double().t() @ y.double()
    torch.testing.assert_close(gram, want, rtol=1e-10, atol=1e-8)
    evals, evecs = stacr_ops.small_eigh(gram)
    ref = torch.linalg.eigvalsh(want).flip(0)
    torch.testing.assert_close(evals, ref, rtol=1e-9, atol=1e-9 * float(ref.abs().max()))
    assert bool((evals[:-1] >= evals[1:]).all())
    recon = evecs @ torch.diag(evals) @ evecs.t()
    assert float((recon - want).abs().max()) < 1e-8 * float(want.abs().max())
    assert float((evecs.t() @ evecs - torch.eye(w, device="cuda", dtype=torch.float64)).abs().max()) < 1e-10


def test_range_finder_without_library_solvers_captures_the_dominant_subspace():
    from stacr_b200.ops.basis import range_finder_basis

    g = torch.Generator(device="cuda").manual_seed(3)
    rows, n, r = 4096, 2048, 8
    u = torch.linalg.qr(torch.randn(n, r, device="cuda", generator=g)).Q
    coeff = torch.randn(rows, r, device="cuda", generator=g) * torch.linspace(10.0, 3.0, r, device="cuda")
    x = (coeff @ u.t() + 0.1 * torch.randn(rows, n, device="cuda", generator=g)).bfloat16()
    q = range_finder_basis(x, r)
    assert float((q.t() @ q - torch.eye(r, device="cuda")).abs().max()) < 1e-3
    captured = float((x.float() @ q).square().sum() / x.float().square().sum())
    best = float((x.float() @ u).square().sum() / x.float().square().sum())
    assert captured > 0.995 * best
