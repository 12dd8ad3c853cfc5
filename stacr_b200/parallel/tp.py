"""Tensor-parallel linears whose collective runs on this library's kernels over symmetric memory.

A Megatron-style block has two all-reduces on its critical path in each direction: the output of the row-parallel
projection in forward and the input gradient of the column-parallel projection in backward.  Both are "GEMM, then
sum over ranks".  Two engines serve them (``STACR_TP_ENGINE``):

* :class:`GemmThenAllReduce` (default): the CTA-pair tensor-core GEMM writes the partial product into a symmetric bf16
  buffer and a bf16 all-reduce kernel sums it in place, in the switch (``multimem.ld_reduce`` with fp32 accumulation +
  ``multimem.st``) or with peer loads and stores.  Any degree up to 16.
* :class:`GemmAllReduce`: ONE tensor-core kernel per rank whose epilogue stores every partial output tile, as whole
  128-byte row segments, into this rank's slot of a staging buffer on *every* rank (``multimem.st`` or peer stores), so
  the transfer of tile i overlaps the math of tile i+1; a second small kernel waits on a flag barrier (bounded) and sums
  the slots locally.  Two staging buffers alternate, so no barrier precedes the GEMM.  Every rank receives ``world``
  tiles per product, which limits it to small degrees, and the remote stores lengthen the GEMM itself; it is kept as
  the measured alternative.

A compressed shard (the projection engine's layer) performs the same collective inside its own forward / input-gradient
product through :class:`TPContext`.

Replaces the ``clone() + dist.all_reduce`` after the row-parallel GEMM and the ``all_reduce`` of the input gradient
of the reference (stacr/protocols/tensor_parallel.py:25-64 there).  Without CUDA, symmetric memory or bf16 operands
the modules fall back to a library GEMM followed by ``torch.distributed.all_reduce``.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..ops import _lib


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


class GemmAllReduce:
    """``sum over ranks of (A_r @ B_r^T)`` with the sum done by the GEMM epilogue over NVLink peer memory."""

    def __init__(self, max_elems: int, device: torch.device, group=None):
        from . import symm

        self.group = group
        world = _world(group)
        self.bufs = [symm.SymmetricBuffer(max_elems * world, torch.bfloat16, device, group) for _ in range(2)]
        for b in self.bufs:
            b.tensor.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.world, self.rank = self.bufs[0].world, self.bufs[0].rank
        self.max_elems, self.device = max_elems, device
        self._peer_lists = [(ctypes.c_ulonglong * 8)(*([int(p) for p in b.peer_ptrs.tolist()] + [0] * (8 - self.world))) for b in self.bufs]
        self.calls = 0
        if self.world > 8:
            raise ValueError("GemmAllReduce supports up to 8 ranks")

    def __call__(self, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias: Optional[torch.Tensor] = None,
                 alpha: float = 1.0) -> torch.Tensor:
        from ..ops.gemm import _pick_bn

        assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(1) == 1 and b.stride(1) == 1
        k, m = a.shape if a_mn else a.shape[::-1]
        n = b.shape[1] if b_mn else b.shape[0]
        if n % 16 or m * n > self.max_elems:
            raise ValueError(f"output {m}x{n} needs N % 16 == 0 and at most {self.max_elems} elements")
        buf = self.bufs[self.calls & 1]
        peers = self._peer_lists[self.calls & 1]
        self.calls += 1
        sms = _lib.sm_count(a.device)
        lib = _lib.load()
        if bias is not None:
            bias = bias.detach().float().contiguous()
        rc = lib.sb_gemm_bf16_allreduce(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(bias), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
            ctypes.c_int(a.stride(0)), ctypes.c_int(b.stride(0)), ctypes.c_int(int(a_mn)), ctypes.c_int(int(b_mn)),
            ctypes.c_int(_pick_bn(m, n, b_mn, sms)), ctypes.c_float(alpha), ctypes.c_int(sms), ctypes.c_int(self.rank), ctypes.c_int(self.world),
            ctypes.c_ulonglong(buf.multicast_ptr if buf.use_multimem else 0), peers, _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_gemm_bf16_allreduce")
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
        flags = self.bufs[0]          # one flag plane and one epoch counter serve both staging buffers
        epoch = flags._next_epoch()
        rc = lib.sb_allreduce_finish(
            _lib.ptr(flags._pad_ptrs), ctypes.c_int(self.rank), ctypes.c_int(self.world), *epoch, _lib.ptr(buf.tensor),
            _lib.ptr(out), ctypes.c_longlong(m), ctypes.c_int(n), ctypes.c_int(max(flags.max_ctas, 32)),
            _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_allreduce_finish")
        _lib.count(2)
        return out


class GemmThenAllReduce:
    """``sum over ranks of (A_r @ B_r^T)`` as two in-tree kernels: the CTA-pair tensor-core GEMM writes its bf16 result into
    a symmetric buffer and the bf16 all-reduce kernel sums it in place over NVLink (in the switch when the fabric has a
    multicast address), after which the result is copied out.  At the sizes of a tensor-parallel GPT-2 block this is
    faster than the single kernel whose epilogue stores every partial tile into every rank (the remote stores stretch a
    24 us GEMM to 53 us at 4096 x 1280 x 2560 on two GPUs), and it works at any degree up to 16."""

    def __init__(self, max_elems: int, device: torch.device, group=None):
        from . import symm

        self.group = group
        self.buf = symm.SymmetricBuffer(max_elems, torch.bfloat16, device, group)
        self.buf.max_ctas = max(self.buf.max_ctas, 16)
        self.world, self.rank, self.max_elems, self.device = self.buf.world, self.buf.rank, max_elems, device

    def __call__(self, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias: Optional[torch.Tensor] = None,
                 alpha: float = 1.0) -> torch.Tensor:
        from ..ops.gemm import gemm

        m = a.shape[1] if a_mn else a.shape[0]
        n = b.shape[1] if b_mn else b.shape[0]
        if (m * n) % 8 or m * n > self.max_elems:
            raise ValueError(f"output {m}x{n} needs a multiple of 8 elements and at most {self.max_elems}")
        out = self.buf.tensor[: m * n].view(m, n)
        gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=None if bias is None else bias.detach().float().contiguous(), out=out, alpha=alpha)
        self.buf.all_reduce_bf16_(0, m * n)
        return out.clone()


_ENGINES: dict = {}


def _max_fused_world() -> int:
    """Largest tensor-parallel degree served by the fused kernel (``STACR_TP_FUSED_MAX_WORLD``, default 2).

    Every rank stores its partial tile into a slot on *every* rank, so each GPU receives ``world`` tiles per GEMM where a
    reduce-scatter + all-gather moves ``2 (world - 1) / world``: the same bytes at degree 2 (where the fused kernel measured
    faster than a library GEMM followed by NCCL), four times as many at degree 8 (where it measured slower).
    """
    import os

    return int(os.environ.get("STACR_TP_FUSED_MAX_WORLD", "2"))


def _engine_kind() -> str:
    """``STACR_TP_ENGINE``: ``pair`` (default) = GEMM kernel + all-reduce kernel over symmetric memory, ``fused`` = the single
    GEMM kernel with the sum in its epilogue (degrees up to ``STACR_TP_FUSED_MAX_WORLD``), ``nccl`` = library collectives."""
    import os

    return os.environ.get("STACR_TP_ENGINE", "pair")


def engine_for(device: torch.device, max_elems: int, group=None):
    """One shared engine per (device, group), grown on demand; ``None`` when the symmetric-memory paths cannot run here."""
    from . import symm

    kind = _engine_kind()
    if _world(group) < 2 or device.type != "cuda" or kind == "nccl" or not symm.available():
        return None
    if kind == "fused" and _world(group) > _max_fused_world():
        kind = "pair"
    key = (device.index, id(group), kind)
    eng = _ENGINES.get(key)
    if eng is None or eng.max_elems < max_elems:
        eng = (GemmAllReduce if kind == "fused" else GemmThenAllReduce)(max(max_elems, 1 << 22), device, group)
        _ENGINES[key] = eng
    return eng


class TPContext:
    """What a compressed linear layer needs to know to act as a tensor-parallel shard.

    ``kind == "row"``: the layer holds input columns; its forward product is a partial sum that has to be added over the
    ranks.  ``kind == "column"``: the layer holds output rows of a replicated input; its input gradient is the partial sum.
    In both cases the compressed layer's own GEMM call is replaced by :meth:`gemm_sum`, which runs the product and the sum
    as one kernel pair over symmetric memory when it can (bf16 CUDA operands, symmetric memory, a supported degree) and
    as GEMM + ``all_reduce`` otherwise.  Activation compression itself is untouched: a row-parallel shard tracks a basis of
    its ``N / tp`` input columns, a column-parallel shard one of the replicated input
    (stacr/protocols/tp_gpt2.py:350-352 of the reference).
    """

    def __init__(self, kind: str, group=None, fused: bool = True):
        if kind not in ("row", "column"):
            raise ValueError("kind must be 'row' or 'column'")
        self.kind, self.group, self.fused = kind, group, fused

    def gemm_sum(self, a: torch.Tensor, b: torch.Tensor, *, b_mn: bool, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``sum over ranks of (a @ b^T [+ bias])`` for bf16 CUDA operands (``b`` is ``[N, K]`` or, with ``b_mn``, ``[K, N]``)."""
        from ..ops.gemm import gemm

        m = a.shape[0]
        n = b.shape[1] if b_mn else b.shape[0]
        eng = None
        if self.fused and n % 16 == 0 and a.shape[1] % 8 == 0:
            eng = engine_for(a.device, m * n, self.group)
        if eng is not None:
            return eng(a, b, b_mn=b_mn, bias=bias)
        y = gemm(a, b, b_mn=b_mn, bias=bias)
        if _world(self.group) > 1:
            dist.all_reduce(y, group=self.group)
        return y

    def sum_(self, t: torch.Tensor) -> torch.Tensor:
        if _world(self.group) > 1:
            t = t.contiguous()
            dist.all_reduce(t, group=self.group)
        return t

    def exact(self, x: torch.Tensor, layer) -> torch.Tensor:
        """The uncompressed path of a wrapped shard (evaluation, frozen weights): plain product plus this shard's collective."""
        w = layer.weight.t() if layer.transposed else layer.weight
        if self.kind == "row":
            y = F.linear(x, w, layer.bias)
            return self.sum_(y) if not torch.is_grad_enabled() else _AllReduceFn.apply(y, self.group)
        if torch.is_grad_enabled() and x.requires_grad:
            x = _CopyFn.apply(x, self.group)
        return F.linear(x, w, layer.bias)


class _AllReduceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, group):
        t = t.clone()
        if _world(group) > 1:
            dist.all_reduce(t, group=group)
        return t

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return t.view_as(t)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if _world(ctx.group) > 1:
            dist.all_reduce(g, group=ctx.group)
        return g, None


def _on_kernels(t: torch.Tensor) -> bool:
    """bf16 CUDA operands (directly or through bf16 autocast): the products of the plain shards run on the in-tree GEMM."""
    if not (t.is_cuda and _lib.available()):
        return False
    return t.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)


def _shard_products(g2d, x2d, weight, need_gx: bool, need_gw: bool, kernels: bool):
    """``(dY W, dY^T X)`` of one shard: in-tree GEMMs on bf16 operands (fp32 weight gradient), framework products otherwise."""
    if kernels and g2d.shape[1] % 8 == 0 and x2d.shape[1] % 8 == 0 and g2d.shape[0] % 8 == 0:
        from ..layers import _bf16_weight
        from ..ops.gemm import gemm

        g = _bf16(g2d).contiguous()
        gx = gemm(g, _bf16_weight(weight).contiguous(), b_mn=True).to(x2d.dtype) if need_gx else None
        gw = gemm(g, _bf16(x2d).contiguous(), a_mn=True, b_mn=True, out_dtype=torch.float32).to(weight.dtype) if need_gw else None
        return gx, gw
    gx = (g2d.to(weight.dtype) @ weight).to(x2d.dtype) if need_gx else None
    gw = (g2d.t().to(x2d.dtype) @ x2d).to(weight.dtype) if need_gw else None
    return gx, gw


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)


class _RowParallelFn(torch.autograd.Function):
    """``y = all_reduce(x_local @ W_local^T) + bias``; no collective in backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, group, engine):
        x2d = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2d, weight)
        ctx.has_bias, ctx.shape = bias is not None, x.shape
        ctx.kernels = _on_kernels(x2d)
        if engine is not None:
            from ..layers import _bf16_weight

            y = engine(_bf16(x2d).contiguous(), _bf16_weight(weight).contiguous(), bias=bias)
        else:
            y = F.linear(x2d, weight.to(x2d.dtype), None if bias is None else bias.to(x2d.dtype))
            if _world(group) > 1:
                dist.all_reduce(y, group=group)
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2d, weight = ctx.saved_tensors
        g2d = gy.reshape(-1, gy.shape[-1])
        gx, gw = _shard_products(g2d, x2d, weight, ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.kernels)
        if gx is not None:
            gx = gx.reshape(ctx.shape)
        gb = g2d.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gx, gw, gb, None, None


class _ColumnParallelFn(torch.autograd.Function):
    """``y = x @ W_local^T + b_local`` on a replicated input; the input gradient is summed over ranks by the GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias, group, engine):
        x2d = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2d, weight)
        ctx.has_bias, ctx.shape, ctx.group, ctx.engine = bias is not None, x.shape, group, engine
        ctx.kernels = _on_kernels(x2d)
        if ctx.kernels and x2d.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0:
            from ..layers import _bf16_weight
            from ..ops.gemm import gemm

            y = gemm(_bf16(x2d).contiguous(), _bf16_weight(weight).contiguous(), bias=None if bias is None else bias.detach().float().contiguous())
        else:
            y = F.linear(x2d, weight.to(x2d.dtype), None if bias is None else bias.to(x2d.dtype))
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2d, weight = ctx.saved_tensors
        g2d = gy.reshape(-1, gy.shape[-1])
        gx = None
        if ctx.needs_input_grad[0]:
            if ctx.engine is not None:
                from ..layers import _bf16_weight

                # dX = dY @ W: W [out_local, in] is the [K, N] operand of this product
                gx = ctx.engine(_bf16(g2d).contiguous(), _bf16_weight(weight).contiguous(), b_mn=True).to(x2d.dtype)
            else:
                gx, _ = _shard_products(g2d, x2d, weight, True, False, ctx.kernels)
                if _world(ctx.group) > 1:
                    dist.all_reduce(gx, group=ctx.group)
            gx = gx.reshape(ctx.shape)
        _, gw = _shard_products(g2d, x2d, weight, False, ctx.needs_input_grad[1], ctx.kernels)
        gb = g2d.sum(0) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gx, gw, gb, None, None


class _FusedBase(nn.Module):
    def __init__(self, linear: nn.Linear, group=None, fused: bool = True):
        super().__init__()
        self.weight, self.bias = linear.weight, linear.bias
        self.in_features, self.out_features = linear.in_features, linear.out_features
        self.group, self.fused = group, fused

    def _engine(self, x: torch.Tensor, out_elems: int) -> Optional[GemmAllReduce]:
        autocast_bf16 = torch.is_autocast_enabled(x.device.type) and torch.get_autocast_dtype(x.device.type) == torch.bfloat16
        if not self.fused or not (x.is_cuda and (x.dtype == torch.bfloat16 or autocast_bf16)):
            return None
        return engine_for(x.device, out_elems, self.group)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, fused={self.fused}"


class RowParallelLinear(_FusedBase):
    """Holds the input-column shard of a projection; ``forward`` returns the full (summed) output on every rank."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.numel() // x.shape[-1]
        ok = self.out_features % 16 == 0 and self.in_features % 8 == 0
        return _RowParallelFn.apply(x, self.weight, self.bias, self.group, self._engine(x, rows * self.out_features) if ok else None)


class ColumnParallelLinear(_FusedBase):
    """Holds the output-row shard of a projection; the input is replicated and its gradient is summed over ranks."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        rows = x.numel() // x.shape[-1]
        ok = self.in_features % 16 == 0 and self.out_features % 8 == 0
        return _ColumnParallelFn.apply(x, self.weight, self.bias, self.group, self._engine(x, rows * self.in_features) if ok else None)


def _fused_engine(x: torch.Tensor, out_elems: int, group) -> Optional[GemmAllReduce]:
    autocast_bf16 = torch.is_autocast_enabled(x.device.type) and torch.get_autocast_dtype(x.device.type) == torch.bfloat16
    if not (x.is_cuda and (x.dtype == torch.bfloat16 or autocast_bf16)):
        return None
    return engine_for(x.device, out_elems, group)


def row_parallel_linear(x: torch.Tensor, linear: nn.Linear, group=None, fused: bool = True) -> torch.Tensor:
    """Functional form of :class:`RowParallelLinear` over an existing ``nn.Linear`` shard."""
    rows = x.numel() // x.shape[-1]
    ok = fused and linear.out_features % 16 == 0 and linear.in_features % 8 == 0
    return _RowParallelFn.apply(x, linear.weight, linear.bias, group, _fused_engine(x, rows * linear.out_features, group) if ok else None)


def column_parallel_linear(x: torch.Tensor, linear: nn.Linear, group=None, fused: bool = True) -> torch.Tensor:
    """Functional form of :class:`ColumnParallelLinear` over an existing ``nn.Linear`` shard."""
    rows = x.numel() // x.shape[-1]
    ok = fused and linear.in_features % 16 == 0 and linear.out_features % 8 == 0
    return _ColumnParallelFn.apply(x, linear.weight, linear.bias, group, _fused_engine(x, rows * linear.in_features, group) if ok else None)
