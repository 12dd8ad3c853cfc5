"""Fused forward primitives on the sm_100a kernels: skinny projection and projection + residual + top-k.

This is the counterpart of the reference project's ``stacr/triton_kernels.py`` (``triton_matmul`` :81-125,
``stacr_forward_fused`` :141-334, ``stacr_forward_pytorch`` :337-396, ``verify_fused_kernel`` :399-466) with the same
function names and return conventions, so code written against that module keeps working
(``stacr_b200.triton_kernels`` is an alias of this module).  Nothing here uses Triton: the projection is the tcgen05
GEMM with a 16/32-wide N tile, and the global top-k is the two-pass radix select that recomputes the residual in
registers and never materialises it.  Differences that a caller can see:

* bf16 is the native operand type (the reference's kernel accepts fp16 only); fp16/fp32 inputs are cast to bf16 on the
  kernel route and the metadata says so;
* ``topk_mode="global"`` runs on the kernels; ``"row"`` (per-row top-k, a dense ``[B, K]`` result) has no kernel and
  uses the chunked framework route, as does anything on the CPU.
"""

from __future__ import annotations

from typing import Tuple

import torch

from .ops import _lib


def kernels_available() -> bool:
    return torch.cuda.is_available() and _lib.available()


def triton_available() -> bool:
    """Kept for callers of the reference API: ``True`` when the in-tree CUDA kernels can run (Triton is never used)."""
    return kernels_available()


def _as_nr(basis: torch.Tensor, n: int) -> torch.Tensor:
    if basis.dim() != 2:
        raise ValueError(f"Expects 2D tensors, got basis {tuple(basis.shape)}")
    if basis.shape[0] == n:
        return basis
    if basis.shape[1] == n:
        return basis.t().contiguous()
    raise ValueError(f"Incompatible shapes: features {n}, basis {tuple(basis.shape)}")


def projection_pytorch(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a.matmul(b)


def triton_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ b [K, N]``; on a B200 with bf16-compatible operands this is the tcgen05 GEMM, else ``torch.matmul``."""
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"Incompatible shapes: {tuple(a.shape)} @ {tuple(b.shape)}")
    if not (kernels_available() and a.is_cuda and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.dtype in (torch.bfloat16, torch.float16)):
        return a.matmul(b)
    from .ops.gemm import gemm

    out = gemm(a.to(torch.bfloat16).contiguous(), b.to(torch.bfloat16).contiguous(), b_mn=True)
    return out.to(a.dtype)


projection_triton = triton_matmul


def stacr_forward_pytorch(input: torch.Tensor, basis: torch.Tensor, budget: float = 0.1, topk_mode: str = "row") -> Tuple:
    """Framework-op reference: ``(coefficients, topk_values, topk_indices)``; values keep their sign."""
    if input.dim() != 2:
        raise ValueError(f"Expects 2D tensors, got input {tuple(input.shape)}")
    b, n = input.shape
    q = _as_nr(basis, n)
    x = input.float() if input.dtype in (torch.float16, torch.bfloat16) else input
    qf = q.to(x.dtype)
    coeff = x @ qf
    residual = x - coeff @ qf.t()
    if topk_mode == "row":
        k = max(1, int(n * budget))
        idx = residual.abs().topk(k, dim=1, sorted=False).indices
        vals = residual.gather(1, idx)
    elif topk_mode == "global":
        k = max(1, int(b * n * budget))
        idx = residual.reshape(-1).abs().topk(k, sorted=False).indices
        vals = residual.reshape(-1)[idx]
    else:
        raise ValueError(f"Unknown topk_mode: {topk_mode}")
    return coeff.to(input.dtype), vals.to(input.dtype), idx


def stacr_forward_fused(input: torch.Tensor, basis: torch.Tensor, budget: float = 0.1, topk_mode: str = "row", chunk_size: int = 512,
                        return_metadata: bool = False) -> Tuple:
    """Projection + residual + top-k without a dense residual tensor.

    Returns ``(coefficients [B, R], topk_values, topk_indices[, metadata])`` with per-row ``[B, K]`` results for
    ``topk_mode="row"`` and flat ``[K]`` results (indices into the flattened ``[B, N]`` tensor) for ``"global"``.
    """
    if input.dim() != 2 or basis.dim() != 2:
        raise ValueError(f"Expects 2D tensors, got input {tuple(input.shape)}, basis {tuple(basis.shape)}")
    if topk_mode not in ("row", "global"):
        raise ValueError(f"Unknown topk_mode: {topk_mode}")
    b, n = input.shape
    q = _as_nr(basis, n)
    r = q.shape[1]
    meta = {"route": "pytorch_chunked", "route_counts": {"pytorch_chunked": 0, "sm100_kernels": 0, "pytorch_fallback": 0}, "parity_error": None,
            "operand_dtype": str(input.dtype)}
    on_kernels = kernels_available() and input.is_cuda and topk_mode == "global" and n % 8 == 0 and r <= 32 and b * n < 2 ** 31 - 1
    if on_kernels:
        from .ops import stacr_ops

        x = input.to(torch.bfloat16).contiguous()
        qb = q.to(torch.bfloat16).contiguous()
        coeff = stacr_ops.project(x, stacr_ops.pad_basis_transpose(qb))[:, :r]
        cb = coeff.to(torch.bfloat16).contiguous()
        k = max(1, int(b * n * budget))
        idx, vals, _scale = stacr_ops.residual_topk(x, cb, qb, [k], b, 0, torch.int32)
        meta["route"] = "sm100_kernels"
        meta["route_counts"]["sm100_kernels"] = 1
        meta["operand_dtype"] = "torch.bfloat16"
        out = (coeff.to(input.dtype), vals.to(input.dtype), idx.long())
        return out + (meta,) if return_metadata else out
    # chunked framework route: the workspace is [chunk_size, N], never [B, N]
    compute = torch.float32 if input.dtype in (torch.float16, torch.bfloat16) else input.dtype
    qf = q.to(compute)
    coeffs, vals, idxs = [], [], []
    for lo in range(0, b, max(1, chunk_size)):
        x = input[lo:lo + chunk_size].to(compute)
        c = x @ qf
        res = x - c @ qf.t()
        coeffs.append(c)
        meta["route_counts"]["pytorch_chunked"] += 1
        if topk_mode == "row":
            k = max(1, int(n * budget))
            i = res.abs().topk(k, dim=1, sorted=False).indices
            vals.append(res.gather(1, i))
            idxs.append(i)
        else:
            k_total = max(1, int(b * n * budget))
            flat = res.reshape(-1)
            kk = min(k_total, flat.numel())
            i = flat.abs().topk(kk, sorted=False).indices
            vals.append(flat[i])
            idxs.append(i + lo * n)
    coeff = torch.cat(coeffs).to(input.dtype)
    if topk_mode == "row":
        out = (coeff, torch.cat(vals).to(input.dtype), torch.cat(idxs))
    else:
        v, i = torch.cat(vals), torch.cat(idxs)
        k_total = max(1, int(b * n * budget))
        if v.numel() > k_total:
            keep = v.abs().topk(k_total, sorted=False).indices
            v, i = v[keep], i[keep]
        out = (coeff, v.to(input.dtype), i)
    return out + (meta,) if return_metadata else out


def verify_fused_kernel(B: int = 64, N: int = 512, R: int = 32, budget: float = 0.1, topk_mode: str = "row") -> bool:
    """Fused route against the framework-op reference on random data: coefficients close, same set of kept positions."""
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=dev).manual_seed(0)
    dtype = torch.bfloat16 if dev == "cuda" else torch.float32
    x = torch.randn(B, N, device=dev, generator=gen).to(dtype)
    q = torch.linalg.qr(torch.randn(N, R, device=dev, generator=gen)).Q.to(dtype)
    c1, v1, i1 = stacr_forward_fused(x, q, budget, topk_mode)
    c0, v0, i0 = stacr_forward_pytorch(x, q, budget, topk_mode)
    if (c1.float() - c0.float()).abs().max() > 3e-2 * max(1.0, float(c0.float().abs().max())):
        return False
    if topk_mode == "row":
        same = torch.equal(i1.sort(dim=1).values, i0.sort(dim=1).values)
    else:
        a, b_ = set(i1.tolist()), set(i0.tolist())
        same = len(a & b_) >= 0.98 * len(b_)          # ties at the threshold and bf16 rounding may swap a few entries
    return bool(same)
