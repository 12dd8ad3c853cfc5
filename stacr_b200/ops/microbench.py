"""Isolated timings of the sm_100a kernels, with roofline fractions against measured peaks.

    python -m stacr_b200.ops.microbench gemm   [--m 8192 --n 8192 --k 2048 --bn 256 --iters 20]
    python -m stacr_b200.ops.microbench stacr  [--rows 8192 --features 8192 --out 2048 --rank 8]
    python -m stacr_b200.ops.microbench optim  [--numel 268435456]
    python -m stacr_b200.ops.microbench attention [--batch 4 --heads 16 --seq 2048 --head-dim 128]

Each case runs warm-up launches, then ``--iters`` timed launches between CUDA events; operands are larger than the
126 MB L2 at the default sizes (the ``stacr`` and ``optim`` cases stream several hundred MB per launch; the default
``gemm`` case reads 160 MB).  ``--iters 1 --warmup 1`` makes a run small enough to sit under a profiler.
Fractions are reported against ``MEASURED_PEAKS.json`` at the repository root when present (fields ``hbm_gbs`` and
``bf16_tflops``) and against 6650 GB/s / 1590 TFLOP/s otherwise; the line says which.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def peaks() -> dict:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.is_file():
        raw = json.loads(path.read_text())
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timed(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def case_gemm(args, pk) -> list:
    from .gemm import gemm

    m, n, k = args.m, args.n, args.k
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    out = []
    flops = 2.0 * m * n * k
    if args.two_cta:
        ref = torch.matmul(a, b.t()).float()
        got = gemm(a, b, two_cta=True).float()
        err = float((got - ref).abs().max() / ref.abs().max())
        ms = timed(lambda: gemm(a, b, two_cta=True), args.iters, args.warmup)
        out.append({"kernel": "gemm2_bf16_kernel (cta_group::2)", "shape": [m, n, k], "ms": ms, "tflops": flops / ms / 1e9, "max_rel_err_vs_cublas": err,
                    f"frac_of_{pk['source']}_bf16": flops / ms / 1e9 / pk["bf16_tflops"]})
    ms = timed(lambda: gemm(a, b, bn=args.bn, two_cta=False), args.iters, args.warmup)
    out.append({"kernel": "gemm_bf16_kernel", "shape": [m, n, k], "bn": args.bn, "ms": ms, "tflops": flops / ms / 1e9,
                f"frac_of_{pk['source']}_bf16": flops / ms / 1e9 / pk["bf16_tflops"]})
    if not args.only_ours:
        ms = timed(lambda: torch.matmul(a, b.t()), args.iters, args.warmup)
        out.append({"kernel": "cublas (torch.matmul)", "shape": [m, n, k], "ms": ms, "tflops": flops / ms / 1e9})
    return out


def case_stacr(args, pk) -> list:
    from . import stacr_ops
    from .basis import oja_step_kernels

    rows, n, o, r = args.rows, args.features, args.out, args.rank
    base = torch.randn(rows, r, device="cuda") @ torch.randn(r, n, device="cuda")
    x = (base + 0.3 * torch.randn(rows, n, device="cuda")).bfloat16()
    del base
    q = torch.linalg.qr(torch.randn(n, r, device="cuda")).Q.contiguous()
    qb = q.bfloat16().contiguous()
    qt = stacr_ops.pad_basis_transpose(qb)
    c = stacr_ops.project(x, qt)[:, :r].bfloat16().contiguous()
    k = int(round(args.budget * rows * n))
    dy = torch.randn(rows, o, device="cuda").bfloat16()
    x_bytes, dy_bytes, dw_bytes = rows * n * 2, rows * o * 2, o * n * 4
    out = []

    def add(name, fn, bytes_moved):
        ms = timed(fn, args.iters, args.warmup)
        out.append({"kernel": name, "shape": [rows, n, o], "ms": ms, "algorithmic_GB": bytes_moved / 1e9, "GBs": bytes_moved / ms / 1e6,
                    f"frac_of_{pk['source']}_hbm": bytes_moved / ms / 1e6 / pk["hbm_gbs"]})

    sel = args.only or ""
    if sel in ("", "project"):
        add("project (gemm_bf16_kernel, N=16)", lambda: stacr_ops.project(x, qt), x_bytes)
    if sel in ("", "topk"):
        add("residual top-k, two exact passes (hist+scan+scale+compact)", lambda: stacr_ops.residual_topk(x, c, qb, [k], rows, 8, torch.int32, sampled=False), 2 * x_bytes)
        add("residual top-k, sampled threshold (sample+candidates+compact)", lambda: stacr_ops.residual_topk(x, c, qb, [k], rows, 8, torch.int32, sampled=True), x_bytes + x_bytes // 16)
        out[-1]["stats"] = stacr_ops.last_sampled_selection_stats()
    if sel in ("", "oja"):
        add("oja_update (+ X^T Y gemm)", lambda: oja_step_kernels(q, x, 0.01), 2 * x_bytes)
    if sel in ("", "gelu"):
        from . import nn_kernels

        h = torch.randn(rows, n, device="cuda").bfloat16()
        g = torch.randn(rows, n, device="cuda").bfloat16()
        add("gelu_fwd", lambda: nn_kernels.gelu_fwd(h, False), 2 * x_bytes)
        add("gelu_bwd + column sums", lambda: nn_kernels.gelu_bwd_colsum(g, h, False), 3 * x_bytes)
        add("colsum (separate pass)", lambda: stacr_ops.colsum(g), x_bytes)
    if sel in ("", "dw"):
        idx, val, scale = stacr_ops.residual_topk(x, c, qb, [k], rows, 8, torch.int32)
        add("weight_grad gather form (bucket + dw_fused)", lambda: stacr_ops.weight_grad(dy, c, q, (idx, val, scale, 8, k), o, n, False, torch.float32, dense=False),
            dy_bytes + dw_bytes + k * o * 2)
        add("weight_grad dense form (rebuild + CTA-pair GEMM)", lambda: stacr_ops.weight_grad(dy, c, q, (idx, val, scale, 8, k), o, n, False, torch.float32, dense=True),
            dy_bytes + dw_bytes + 2 * x_bytes)
        out[-1]["TFLOPs"] = 2.0 * rows * n * o / out[-1]["ms"] / 1e9
        add("rebuild_input (C Q^T + S in bf16)", lambda: stacr_ops.rebuild_input(c, q, (idx, val, scale, 8, k), rows, n), x_bytes)
        add("weight_grad low-rank only", lambda: stacr_ops.weight_grad(dy, c, q, None, o, n, False, torch.float32), dy_bytes + dw_bytes)
    return out


def case_optim(args, pk) -> list:
    from ..optim import AdamW8bit

    p = torch.nn.Parameter(torch.randn(args.numel, device="cuda"))
    p.grad = torch.randn_like(p) * 1e-3
    opt = AdamW8bit([p], lr=1e-4, bf16_shadow=True)
    ms = timed(opt.step, args.iters, args.warmup)
    moved = args.numel * (4 + 4 + 4 + 2 + 2 + 2 + 2)  # param r/w, grad r, 8-bit m and v r/w, bf16 shadow w
    return [{"kernel": "adamw_8bit_kernel", "numel": args.numel, "ms": ms, "algorithmic_GB": moved / 1e9, "GBs": moved / ms / 1e6,
             f"frac_of_{pk['source']}_hbm": moved / ms / 1e6 / pk["hbm_gbs"]}]


def case_attention(args, pk) -> list:
    """The in-tree flash-attention forward against the library kernel on views of a fused, per-head interleaved QKV matrix."""
    import torch.nn.functional as F

    from . import attention

    b, h, s, d = args.batch, args.heads, args.seq, args.head_dim
    qkv = torch.randn(b * s, h * 3 * d, device="cuda").bfloat16()
    q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, h, 3 * d).split(d, dim=-1))
    causal = not args.full
    flops = 4.0 * b * h * s * s * d * (0.5 if causal else 1.0)
    rows = []
    ms = timed(lambda: attention.forward(q, k, v, causal=causal), args.iters, args.warmup)
    rows.append({"kernel": "flash_fwd_kernel (in-tree)", "shape": [b, h, s, d], "causal": causal, "ms": ms, "TFLOPs": flops / ms / 1e9,
                 f"frac_of_{pk['source']}_bf16": flops / ms / 1e9 / pk["bf16_tflops"]})
    if d == 128:
        out, lse = attention.forward(q, k, v, causal=causal)
        dout = torch.randn(b, s, h * d, device="cuda").bfloat16()
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = (t.transpose(1, 2) for t in dqkv.view(b, s, h, 3 * d).split(d, dim=-1))
        ms = timed(lambda: attention.backward(q, k, v, out, dout, lse, dq, dk, dv, causal=causal), args.iters, args.warmup)
        rows.append({"kernel": "flash_bwd_kernel + delta + dq convert (in-tree)", "shape": [b, h, s, d], "causal": causal, "ms": ms,
                     "TFLOPs": 2.5 * flops / ms / 1e9})
        if not args.only_ours:
            ql, kl, vl = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
            ol = F.scaled_dot_product_attention(ql, kl, vl, is_causal=causal)
            gl = dout.view(b, s, h, d).transpose(1, 2)
            ms = timed(lambda: torch.autograd.grad(ol, (ql, kl, vl), gl, retain_graph=True), args.iters, args.warmup)
            rows.append({"kernel": "scaled_dot_product_attention backward (library)", "shape": [b, h, s, d], "causal": causal, "ms": ms,
                         "TFLOPs": 2.5 * flops / ms / 1e9})
    if not args.only_ours:
        ms = timed(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=causal), args.iters, args.warmup)
        rows.append({"kernel": "scaled_dot_product_attention (library)", "shape": [b, h, s, d], "causal": causal, "ms": ms, "TFLOPs": flops / ms / 1e9})
        mine, _ = attention.forward(q, k, v, causal=causal)
        ref = F.scaled_dot_product_attention(q, k, v, is_causal=causal).transpose(1, 2).reshape(b, s, h * d)
        rows[0]["max_abs_diff_vs_library"] = float((mine.float() - ref.float()).abs().max())
    return rows


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=("gemm", "stacr", "optim", "attention"))
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--m", type=int, default=8192)
    parser.add_argument("--n", type=int, default=8192)
    parser.add_argument("--k", type=int, default=2048)
    parser.add_argument("--bn", type=int, default=256)
    parser.add_argument("--only-ours", action="store_true")
    parser.add_argument("--two-cta", action="store_true", help="also run the CTA-pair kernel and check it against the library")
    parser.add_argument("--rows", type=int, default=8192)
    parser.add_argument("--features", type=int, default=8192)
    parser.add_argument("--out", type=int, default=2048)
    parser.add_argument("--rank", type=int, default=8)
    parser.add_argument("--budget", type=float, default=0.005)
    parser.add_argument("--only", choices=("project", "topk", "oja", "dw", "gelu"))
    parser.add_argument("--numel", type=int, default=1 << 28)
    parser.add_argument("--batch", type=int, default=4)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--seq", type=int, default=2048)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--full", action="store_true", help="attention case: no causal mask")
    args = parser.parse_args(argv)
    from . import _lib

    pk = peaks()
    rows = {"gemm": case_gemm, "stacr": case_stacr, "optim": case_optim, "attention": case_attention}[args.case](args, pk)
    _lib.check_status()
    for row in rows:
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
