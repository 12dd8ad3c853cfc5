"""Factorisation comparators: truncated SVD, tensor-train (TT-SVD) and Tucker (HOSVD), with int8/int4 factors.

The decompositions are implemented directly on ``torch.linalg`` (no third-party tensor library): TT-SVD is the
sequential truncated SVD of the unfoldings, Tucker is the higher-order SVD with mode-wise factor matrices and
a projected core.  Parity: stacr/protocols/compression.py:12-718 of the reference project.
"""

from __future__ import annotations

import math
import time
from contextlib import nullcontext

import torch

from .reshape import Reshaper


def _unfold(t: torch.Tensor, mode: int) -> torch.Tensor:
    return t.movedim(mode, 0).reshape(t.shape[mode], -1)


def _mode_dot(t: torch.Tensor, m: torch.Tensor, mode: int) -> torch.Tensor:
    """Contract ``m`` (``J x I_mode``) with mode ``mode`` of ``t``."""
    moved = t.movedim(mode, 0)
    out = (m @ moved.reshape(moved.shape[0], -1)).reshape(m.shape[0], *moved.shape[1:])
    return out.movedim(0, mode)


class Compressor:
    """Static helpers; every ``compress_*_factors`` returns plain tensors that ``decompress_*`` inverts."""

    # ------------------------------------------------------------------ validation
    @staticmethod
    def _normalize_reshape_shape(matrix, reshape_shape):
        shape = tuple(int(d) for d in reshape_shape)
        if math.prod(shape) != matrix.numel():
            raise ValueError(f"reshape_shape {shape} does not match {tuple(matrix.shape)}")
        return shape

    @staticmethod
    def _validate_inputs(matrix, reshape_shape=None, rank=None, variance_threshold=None):
        if not isinstance(matrix, torch.Tensor) or matrix.dim() < 2:
            raise ValueError("matrix must be a tensor with at least two dimensions")
        if not torch.isfinite(matrix).all():
            raise ValueError("matrix must be finite")
        if rank is not None and (isinstance(rank, bool) or int(rank) < 1):
            raise ValueError("rank must be a positive integer")
        if variance_threshold is not None and not 0 < variance_threshold <= 1:
            raise ValueError("variance_threshold must be in (0, 1]")
        if reshape_shape is not None:
            Compressor._normalize_reshape_shape(matrix, reshape_shape)

    @staticmethod
    def _prepare_decomposition_input(tensor):
        return tensor.detach().float() if tensor.dtype in (torch.float16, torch.bfloat16) else tensor.detach()

    @staticmethod
    def _decomposition_context(device):
        return torch.autocast(device_type=torch.device(device).type, enabled=False) if torch.device(device).type in ("cuda", "cpu") else nullcontext()

    # ------------------------------------------------------------------ SVD
    @staticmethod
    def get_rank_from_variance(eigenvalues, threshold):
        energy = torch.cumsum(eigenvalues, 0) / eigenvalues.sum().clamp_min(1e-30)
        hits = (energy >= threshold).nonzero()
        return int(hits[0]) + 1 if hits.numel() else int(eigenvalues.numel())

    @staticmethod
    def compress_svd_factors(matrix, rank, profile: bool = False, use_lowrank: bool = False):
        Compressor._validate_inputs(matrix, rank=rank)
        x = Compressor._prepare_decomposition_input(matrix.reshape(matrix.shape[0], -1))
        t0 = time.perf_counter()
        with Compressor._decomposition_context(x.device):
            r = min(int(rank), *x.shape)
            if use_lowrank and min(x.shape) > 4 * r:
                u, s, v = torch.svd_lowrank(x, q=min(min(x.shape), r + 4), niter=2)
                u, s, vh = u[:, :r], s[:r], v[:, :r].t()
            else:
                u, s, vh = torch.linalg.svd(x, full_matrices=False)
                u, s, vh = u[:, :r], s[:r], vh[:r]
        factors = (u.contiguous(), s.contiguous(), vh.contiguous())
        return (factors, {"seconds": time.perf_counter() - t0}) if profile else factors

    @staticmethod
    def compress_svd(matrix, variance_threshold=0.9, rank=None):
        Compressor._validate_inputs(matrix, variance_threshold=variance_threshold)
        x = Compressor._prepare_decomposition_input(matrix.reshape(matrix.shape[0], -1))
        u, s, vh = torch.linalg.svd(x, full_matrices=False)
        r = int(rank) if rank else Compressor.get_rank_from_variance(s.square(), variance_threshold)
        return u[:, :r].contiguous(), s[:r].contiguous(), vh[:r].contiguous()

    @staticmethod
    def decompress_svd(factors, profile: bool = False):
        u, s, vh = factors
        t0 = time.perf_counter()
        out = (u * s) @ vh
        return (out, {"seconds": time.perf_counter() - t0}) if profile else out

    # ------------------------------------------------------------------ Tucker (HOSVD)
    @staticmethod
    def compress_tucker_factors(matrix, reshape_shape, ranks, profile: bool = False):
        Compressor._validate_inputs(matrix, reshape_shape=reshape_shape)
        t = Reshaper.to_tensor(Compressor._prepare_decomposition_input(matrix), reshape_shape)
        ranks = [max(1, min(int(r), d)) for r, d in zip(ranks, t.shape)]
        t0 = time.perf_counter()
        factors = []
        with Compressor._decomposition_context(t.device):
            for mode, r in enumerate(ranks):
                u = torch.linalg.svd(_unfold(t, mode), full_matrices=False).U[:, :r]
                factors.append(u.contiguous())
            core = t
            for mode, u in enumerate(factors):
                core = _mode_dot(core, u.t(), mode)
        data = {"core": core.contiguous(), "factors": factors, "shape": tuple(matrix.shape)}
        return (data, {"seconds": time.perf_counter() - t0}) if profile else data

    @staticmethod
    def compress_tucker(matrix, reshape_shape, variance_threshold=0.9):
        Compressor._validate_inputs(matrix, reshape_shape=reshape_shape, variance_threshold=variance_threshold)
        t = Reshaper.to_tensor(Compressor._prepare_decomposition_input(matrix), reshape_shape)
        ranks = [Compressor.get_rank_from_variance(torch.linalg.svdvals(_unfold(t, m)).square(), variance_threshold) for m in range(t.dim())]
        return Compressor.compress_tucker_factors(matrix, reshape_shape, ranks)

    @staticmethod
    def decompress_tucker(compressed_data, profile: bool = False):
        t0 = time.perf_counter()
        out = compressed_data["core"]
        for mode, u in enumerate(compressed_data["factors"]):
            out = _mode_dot(out, u, mode)
        out = out.reshape(compressed_data["shape"])
        return (out, {"seconds": time.perf_counter() - t0}) if profile else out

    # ------------------------------------------------------------------ tensor train (TT-SVD)
    @staticmethod
    def compress_tt_factors(matrix, reshape_shape, rank, profile: bool = False):
        Compressor._validate_inputs(matrix, reshape_shape=reshape_shape, rank=rank)
        t = Reshaper.to_tensor(Compressor._prepare_decomposition_input(matrix), reshape_shape)
        dims = list(t.shape)
        t0 = time.perf_counter()
        cores, r_prev, rest = [], 1, t.reshape(1, -1)
        with Compressor._decomposition_context(t.device):
            for d in dims[:-1]:
                rest = rest.reshape(r_prev * d, -1)
                u, s, vh = torch.linalg.svd(rest, full_matrices=False)
                r = max(1, min(int(rank), s.numel()))
                cores.append(u[:, :r].reshape(r_prev, d, r).contiguous())
                rest = (s[:r, None] * vh[:r])
                r_prev = r
            cores.append(rest.reshape(r_prev, dims[-1], 1).contiguous())
        data = {"cores": cores, "shape": tuple(matrix.shape)}
        return (data, {"seconds": time.perf_counter() - t0}) if profile else data

    @staticmethod
    def compress_tt(matrix, reshape_shape, rank_preset=10):
        return Compressor.compress_tt_factors(matrix, reshape_shape, rank_preset)

    @staticmethod
    def decompress_tt(factors, profile: bool = False):
        t0 = time.perf_counter()
        cores = factors["cores"]
        out = cores[0].reshape(cores[0].shape[1], cores[0].shape[2])
        for core in cores[1:]:
            out = (out @ core.reshape(core.shape[0], -1)).reshape(-1, core.shape[2])
        out = out.reshape(factors["shape"])
        return (out, {"seconds": time.perf_counter() - t0}) if profile else out

    # ------------------------------------------------------------------ factor quantisation
    @staticmethod
    def _quantize_tensor_int8(tensor):
        amax = tensor.abs().amax().float()
        scale = (amax / 127.0).clamp_min(torch.finfo(torch.float32).tiny)
        return torch.round(tensor.float() / scale).clamp_(-127, 127).to(torch.int8), scale

    @staticmethod
    def _dequantize_tensor_int8(quantized, scale):
        return quantized.float() * scale

    @staticmethod
    def _quantize_tensor_int4(tensor):
        flat = tensor.reshape(-1).float()
        scale = (flat.abs().amax() / 7.0).clamp_min(torch.finfo(torch.float32).tiny)
        q = (torch.round(flat / scale).clamp_(-7, 7) + 8).to(torch.uint8)
        if q.numel() & 1:
            q = torch.nn.functional.pad(q, (0, 1), value=8)
        pairs = q.view(-1, 2)
        return pairs[:, 0] | (pairs[:, 1] << 4), scale, tuple(tensor.shape), tensor.numel()

    @staticmethod
    def _dequantize_tensor_int4(packed, scale, orig_shape, orig_numel):
        nib = torch.stack((packed & 0x0F, (packed >> 4) & 0x0F), dim=1).reshape(-1)[:orig_numel]
        return ((nib.to(torch.int8) - 8).float() * scale).reshape(orig_shape)

    @staticmethod
    def _q(tensor, bits):
        if bits == 8:
            q, s = Compressor._quantize_tensor_int8(tensor)
            return {"bits": 8, "data": q, "scale": s, "dtype": tensor.dtype}
        if bits == 4:
            q, s, shape, n = Compressor._quantize_tensor_int4(tensor)
            return {"bits": 4, "data": q, "scale": s, "shape": shape, "numel": n, "dtype": tensor.dtype}
        raise ValueError("bits must be 4 or 8")

    @staticmethod
    def _dq(entry):
        if entry["bits"] == 8:
            return Compressor._dequantize_tensor_int8(entry["data"], entry["scale"]).to(entry["dtype"])
        return Compressor._dequantize_tensor_int4(entry["data"], entry["scale"], entry["shape"], entry["numel"]).to(entry["dtype"])

    @staticmethod
    def quantize_svd_factors(factors, bits=8):
        return {"method": "svd", "tensors": [Compressor._q(f, bits) for f in factors]}

    @staticmethod
    def dequantize_svd_factors(quantized_factors):
        return tuple(Compressor._dq(e) for e in quantized_factors["tensors"])

    @staticmethod
    def quantize_tt_factors(factors, bits=8):
        return {"method": "tt", "shape": factors["shape"], "tensors": [Compressor._q(c, bits) for c in factors["cores"]]}

    @staticmethod
    def dequantize_tt_factors(quantized_factors):
        return {"cores": [Compressor._dq(e) for e in quantized_factors["tensors"]], "shape": quantized_factors["shape"]}

    @staticmethod
    def quantize_tucker_factors(factors, bits=8):
        return {"method": "tucker", "shape": factors["shape"], "core": Compressor._q(factors["core"], bits),
                "tensors": [Compressor._q(f, bits) for f in factors["factors"]]}

    @staticmethod
    def dequantize_tucker_factors(quantized_factors):
        return {"core": Compressor._dq(quantized_factors["core"]), "factors": [Compressor._dq(e) for e in quantized_factors["tensors"]],
                "shape": quantized_factors["shape"]}

    @staticmethod
    def get_quantized_storage_bytes(quantized_factors):
        entries = list(quantized_factors["tensors"]) + ([quantized_factors["core"]] if "core" in quantized_factors else [])
        return sum(e["data"].numel() * e["data"].element_size() + 4 for e in entries)

    @staticmethod
    def get_memory_usage(obj):
        if isinstance(obj, torch.Tensor):
            return obj.numel() * obj.element_size()
        if isinstance(obj, dict):
            return sum(Compressor.get_memory_usage(v) for v in obj.values())
        if isinstance(obj, (list, tuple)):
            return sum(Compressor.get_memory_usage(v) for v in obj)
        return 0
