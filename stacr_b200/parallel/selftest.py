"""Multi-GPU self-test of the symmetric-memory all-reduce kernels.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m stacr_b200.parallel.selftest

Each rank fills a symmetric buffer with rank-dependent values, reduces slices of it with the
two-shot peer kernel and (when the fabric exposes a multicast address) the multimem kernel, and
compares with ``torch.distributed.all_reduce`` on a copy.  Also times both against NCCL with CUDA
events (max over ranks).  Prints one JSON line from rank 0 and exits non-zero on a mismatch.
"""

from __future__ import annotations

import json
import sys

import torch
import torch.distributed as dist

from ..ops import _lib
from . import symm
from .ddp import init_distributed


def _time(fn, iters=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _kernel_times(fn, iters=10) -> dict:
    """Mean device time per kernel name (microseconds) over `iters` calls, from the profiler's kernel records."""
    from torch.profiler import ProfilerActivity, profile

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
    out = {}
    for e in prof.key_averages():
        t = getattr(e, "device_time_total", None) or getattr(e, "cuda_time_total", 0)
        if t:
            out[e.key[:60]] = round(t / iters, 2)
    return out


def _fused_dw_check(buf, rank, world, dev, report) -> bool:
    """Weight-gradient kernel with the reduce-scatter in its epilogue + all-gather of owner slices vs NCCL all-reduce."""
    from ..ops import stacr_ops

    class Sink:
        pass

    rows, n_in, n_out, r = 2048, 1024, 1536, 8
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = (torch.randn(rows, r, device=dev, generator=gen) @ torch.randn(r, n_in, device=dev, generator=gen)
         + 0.3 * torch.randn(rows, n_in, device=dev, generator=gen)).bfloat16()
    q = torch.linalg.qr(torch.randn(n_in, r, device=dev, generator=gen)).Q.contiguous()
    qb = q.bfloat16().contiguous()
    c = stacr_ops.project(x, stacr_ops.pad_basis_transpose(qb))[:, :r].bfloat16().contiguous()
    k = int(round(0.005 * rows * n_in))
    res = stacr_ops.residual_topk(x, c, qb, [k], rows, 8, torch.int32) + (8, k)
    dy = torch.randn(rows, n_out, device=dev, generator=gen).bfloat16()
    want = stacr_ops.weight_grad(dy, c, q, res, n_out, n_in, False, torch.float32)
    dist.all_reduce(want)
    want /= world
    off, numel = 4096, n_out * n_in
    good = True
    for mm in ([False, True] if buf.multicast_ptr else [False]):
        buf.use_multimem = mm
        buf.tensor.zero_()
        buf.barrier()                      # every copy is cleared before any rank adds into it
        sink = Sink()
        sink.flat, sink.mode, sink.scale, sink.param_off, sink.region_lo, sink.world = buf.tensor, 2, 1.0, off, off, world
        sink.per_vecs, sink.peer_ptrs = buf.slice_vecs(off, off + numel), buf.peer_ptrs
        stacr_ops.weight_grad(dy, c, q, res, n_out, n_in, False, torch.float32, sink=sink)
        buf.all_gather_slices_(off, off + numel, average=True)
        torch.cuda.synchronize()
        _lib.check_status(dev)
        err = float((buf.tensor[off:off + numel].view_as(want) - want).abs().max())
        clean = float(buf.tensor[:off].abs().max()) == 0.0 and float(buf.tensor[off + numel:off + numel + 4096].abs().max()) == 0.0
        report[f"fused_dw_{'multimem' if mm else 'p2p'}_max_err"] = err
        good &= err < 1e-4 * max(1.0, float(want.abs().max())) and clean
        dist.barrier()
    return good


def _tp_gemm_check(rank, world, dev, report) -> bool:
    """Both tensor-parallel engines (single kernel with the sum in the epilogue; GEMM kernel + bf16 all-reduce kernel) against
    a library GEMM + NCCL all-reduce (shapes of a GPT-2-large block at TP degree `world`)."""
    from .tp import GemmAllReduce, GemmThenAllReduce

    m, n, k = 4096, 1280, 5120 // world
    gen = torch.Generator(device=dev).manual_seed(500 + rank)
    a = (torch.randn(m, k, device=dev, generator=gen) / 8).bfloat16()
    w = (torch.randn(n, k, device=dev, generator=gen) / 8).bfloat16()
    bias = torch.randn(n, device=dev, generator=gen) if rank == 0 else None
    want = a.float() @ w.float().t()
    if bias is not None:
        want += bias
    dist.all_reduce(want)
    good = True
    engines = [("pair", GemmThenAllReduce(m * n, dev))]
    if world <= 8:
        engines.append(("fused", GemmAllReduce(m * n, dev)))
    for label, eng in engines:
        bufs = eng.bufs if label == "fused" else [eng.buf]
        for mm in ([False, True] if bufs[0].multicast_ptr else [False]):
            for b in bufs:
                b.use_multimem = mm
            for _ in range(3):                       # three calls: buffer reuse (and, for the fused engine, both staging buffers) is exercised
                got = eng(a, w, bias=bias)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            err = float((got.float() - want).abs().max() / want.abs().max())
            name = f"{label}_{'multimem' if mm else 'p2p'}"
            report[f"tp_gemm_allreduce_{name}_rel_err"] = err
            good &= err < 2e-2                       # bf16 partial sums
            report[f"tp_gemm_allreduce_{name}_ms"] = _time(lambda: eng(a, w, bias=bias), iters=20)
            report[f"tp_gemm_allreduce_{name}_kernel_us"] = _kernel_times(lambda: eng(a, w, bias=bias))
    report["tp_gemm_allreduce_p2p_rel_err"] = report.get("tp_gemm_allreduce_fused_p2p_rel_err", report["tp_gemm_allreduce_pair_p2p_rel_err"])

    def library():
        y = torch.nn.functional.linear(a, w)
        dist.all_reduce(y)
        return y

    report["tp_gemm_then_nccl_ms"] = _time(library, iters=20)
    report["tp_gemm_then_nccl_kernel_us"] = _kernel_times(library)
    report["tp_gemm_alone_ms"] = _time(lambda: torch.nn.functional.linear(a, w), iters=20)
    report["tp_shape"] = [m, n, k]
    return good


def _reduce_to_owner_check(buf, rank, world, dev, report) -> bool:
    """Reduce-to-owner kernel (peer loads and in-switch reduction) against NCCL all-reduce on the owner's slice; the rest of
    the range must keep its local values."""
    good = True
    n = 1 << 22
    for name, mm in [("p2p", False)] + ([("multimem", True)] if buf.multicast_ptr else []):
        buf.use_multimem = mm
        for lo, hi in ((0, 2048 * world * 4), (4096, 4096 + 2048 * world * 37)):
            gen = torch.Generator(device=dev).manual_seed(31 * rank + lo)
            buf.tensor[:n].copy_(torch.randn(n, device=dev, generator=gen))
            before = buf.tensor[:n].clone()
            expect = before[lo:hi].clone()
            torch.cuda.synchronize()
            dist.barrier()
            dist.all_reduce(expect)
            expect /= world
            per = (hi - lo) // world
            a, b = lo + rank * per, lo + (rank + 1) * per
            buf.reduce_to_owner_(lo, hi, a, b, average=True)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            err = float((buf.tensor[a:b] - expect[a - lo:b - lo]).abs().max())
            same = torch.equal(buf.tensor[:a], before[:a]) and torch.equal(buf.tensor[b:n], before[b:n])
            report[f"reduce_to_owner_{name}_max_err"] = max(err, report.get(f"reduce_to_owner_{name}_max_err", 0.0))
            good &= err < 1e-5 and same
            dist.barrier()
    return good


def _sharded_optimizer_check(rank, world, dev, report) -> bool:
    """A small decoder trained for a few steps with the replicated and with the sharded optimizer: same losses, same bf16
    weights on every rank (the sharded path publishes them through the multicast stores of the update kernel)."""
    import stacr_b200 as S
    from ..models import GPTNeoXForCausalLM, NeoXConfig
    from ..optim import AdamW8bit
    from .ddp import GradSync, broadcast_parameters
    from .zero import ShardedGradSync

    cfg = NeoXConfig(vocab_size=2048, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=1024, max_position_embeddings=128)

    def run(sharded: bool):
        torch.manual_seed(7)
        model = GPTNeoXForCausalLM(cfg).to(dev).train()
        broadcast_parameters(model)
        layers = S.apply_stacr(model, rank=8, residual_budget=0.01, residual_mode="global_topk", turbo_after_step=None, min_features=128)
        if sharded:
            sync = ShardedGradSync(model.parameters(), bucket_mb=1.0)
            opt = AdamW8bit(model.parameters(), lr=1e-3, weight_decay=0.0, bf16_shadow=True, shard=sync)
        else:
            sync = GradSync(model.parameters(), bucket_mb=1.0)
            opt = AdamW8bit(model.parameters(), lr=1e-3, weight_decay=0.0, bf16_shadow=True)
        gen = torch.Generator(device=dev).manual_seed(50 + rank)
        losses = []
        for step in range(5):
            ids = torch.randint(0, cfg.vocab_size, (4, 128), device=dev, generator=gen)
            S.set_step(layers, step)
            sync.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model(input_ids=ids, labels=ids).loss
            loss.backward()
            sync.finish()
            opt.step()
            losses.append(float(loss))
        torch.cuda.synchronize()
        _lib.check_status(dev)
        if sharded:
            sync.gather_parameters()
        weights = {n: p.detach().clone() for n, p in model.named_parameters()}
        shadows = {n: p._bf16_shadow.detach().clone() for n, p in model.named_parameters() if getattr(p, "_bf16_shadow", None) is not None}
        sync.close()
        opt.close()
        return losses, weights, shadows

    la, wa, sa = run(False)
    lb, wb, sb = run(True)
    loss_gap = max(abs(a - b) for a, b in zip(la, lb))
    # The two runs differ in the last bits of every gradient (atomics, tie-breaks in the selection) and Adam turns a sign
    # flip of a near-zero gradient into a full-size step, so the weights are compared as update directions of the matrices.
    torch.manual_seed(7)
    start = {n: p.detach().clone() for n, p in GPTNeoXForCausalLM(cfg).to(dev).named_parameters()}
    cosines = []
    for n in sb:
        ua, ub = (wa[n] - start[n]).reshape(-1).double(), (wb[n] - start[n]).reshape(-1).double()
        cosines.append(float(torch.dot(ua, ub) / (ua.norm() * ub.norm() + 1e-30)))
    update_cos = min(cosines)
    # after gather_parameters the masters of the sharded run round to exactly the published bf16 weights
    master_gap = max(float((wb[n].to(torch.bfloat16).float() - sb[n].float()).abs().max()) for n in sb)
    # every rank must hold the same bf16 weights after the sharded run
    digest = torch.stack([v.float().sum() for v in sb.values()])
    lo, hi = digest.clone(), digest.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    spread = float((hi - lo).abs().max())
    report.update(sharded_loss_gap=loss_gap, sharded_update_cosine=update_cos, sharded_master_vs_bf16_gap=master_gap, sharded_rank_spread=spread,
                  sharded_losses=lb)
    return loss_gap < 5e-2 and update_cos > 0.8 and master_gap == 0.0 and spread == 0.0


def main() -> int:
    rank, world, local = init_distributed("nccl")
    dev = torch.device("cuda", local)
    report = {"world": world, "available": symm.available()}
    if world < 2 or not symm.available():
        if rank == 0:
            print(json.dumps(report))
        return 0
    n = 64 * 1024 * 1024  # 256 MB of fp32
    buf = symm.SymmetricBuffer(n, torch.float32, dev)
    report["multicast"] = buf.multicast_ptr != 0
    ok = True
    modes = [("two_shot", False)] + ([("multimem", True)] if buf.multicast_ptr else [])
    for name, mm in modes:
        buf.use_multimem = mm
        for lo, hi in ((0, 4096), (1024, 1024 + 1000 * 4), (0, n), (n // 2 + 8, n - 4)):
            gen = torch.Generator(device=dev).manual_seed(17 * rank + lo)
            buf.tensor.copy_(torch.randn(n, device=dev, generator=gen))
            expect = buf.tensor[lo:hi].clone()
            torch.cuda.synchronize()
            dist.barrier()
            dist.all_reduce(expect)
            expect /= world
            untouched = buf.tensor[:lo].clone(), buf.tensor[hi:].clone()
            buf.all_reduce_(lo, hi, average=True)
            torch.cuda.synchronize()
            _lib.check_status(dev)
            err = float((buf.tensor[lo:hi] - expect).abs().max())
            same = torch.equal(buf.tensor[:lo], untouched[0]) and torch.equal(buf.tensor[hi:], untouched[1])
            good = err < 1e-5 and same
            ok &= good
            if rank == 0 and not good:
                report.setdefault("failures", []).append({"mode": name, "lo": lo, "hi": hi, "err": err, "outside_untouched": same})
            dist.barrier()
        for ctas in (16, 32, 64, 128):
            buf.max_ctas = ctas
            ms = _time(lambda: buf.all_reduce_(0, n, average=False))
            report[f"{name}_ms_256MB_{ctas}ctas"] = ms
            report[f"{name}_busbw_GBs_{ctas}ctas"] = 2 * (world - 1) / world * n * 4 / ms / 1e6
        buf.max_ctas = 32
    ok &= _fused_dw_check(buf, rank, world, dev, report)
    ok &= _reduce_to_owner_check(buf, rank, world, dev, report)
    ok &= _tp_gemm_check(rank, world, dev, report)
    ok &= _sharded_optimizer_check(rank, world, dev, report)
    plain = torch.randn(n, device=dev)
    ms = _time(lambda: dist.all_reduce(plain))
    report["nccl_ms_256MB"] = ms
    report["nccl_busbw_GBs"] = 2 * (world - 1) / world * n * 4 / ms / 1e6
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    report["ok"] = bool(flag.item())
    if rank == 0:
        print(json.dumps(report), flush=True)
    dist.destroy_process_group()
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
