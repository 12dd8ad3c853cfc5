"""Headline benchmark: full STAC-R training step of a Pythia-1.4B-shaped decoder, tokens/s over N GPUs.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N --steps K ...   # the unmodified reference package

Config (both arms): 24 layers, d_model 2048, 16 heads, MLP 8192, rotary on 25 % of head dims,
parallel attention+MLP residual, vocab 50304, seq 2048, batch 4 per GPU, bf16 compute, random
init, uniform-random tokens; STAC-R on the MLP surface with rank 8, residual budget 0.005,
residual_mode=global_topk, no turbo; AdamW with 8-bit block-wise moments (this framework) --
the reference arm uses torch AdamW because the external 8-bit optimizer it relies on is not
installed; data-parallel over N ranks (weak scaling).

Two measurements, each the median of ``--repeats`` back-to-back timed regions of K optimizer steps
(every region bracketed by barrier + synchronize and timed with CUDA events, max over ranks):
(1) device-resident inputs, no host read-back -> ``value``; (2) end to end through the public API,
with the step's token batch copied from pinned host memory and the loss read back every step ->
``e2e``.  After the timed regions eight extra passes (one per synthetic batch) measure, for both arms alike, the cosine of every
wrapped layer's weight gradient to the dense ``dY^T X`` and the bytes autograd actually saved inside
the wrapped layers.  One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
# keep stdout to the one JSON line: NCCL prints its version banner to stdout at the VERSION/INFO levels
if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
    os.environ["NCCL_DEBUG"] = "WARN"

MODEL = dict(vocab_size=50304, hidden_size=2048, num_hidden_layers=24, num_attention_heads=16, intermediate_size=8192,
             rotary_pct=0.25, max_position_embeddings=2048, use_parallel_residual=True)
SEQ, BATCH = 2048, 4
STACR = dict(rank=8, residual_budget=0.005, residual_mode="global_topk", turbo_after_step=None, surface="mlp", min_features=256)
SMALL = dict(vocab_size=8192, hidden_size=512, num_hidden_layers=4, num_attention_heads=8, intermediate_size=2048,
             rotary_pct=0.25, max_position_embeddings=512, use_parallel_residual=True)


# ----------------------------------------------------------------------------------- harness
class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) > 8 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        power = [float(r[3]) for r in self.rows if len(r) > 8 and r[3].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "power_w_max": max(power) if power else None, "samples": len(self.rows)}


def timed_region(torch, dist, steps, step_fn, world):
    """Barrier + sync, K steps between CUDA events, sync + barrier; returns max-over-ranks seconds."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    secs = torch.tensor([e0.elapsed_time(e1) / 1e3], device="cuda")
    if world > 1:
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(secs)


def fidelity_and_saved_bytes(torch, model, layers, run_forward_backward):
    """Evidence gathered by one extra forward + backward pass outside every timed region, identically for both arms.

    * Saved bytes, measured: while a wrapped layer's forward runs, every tensor autograd saves that is not a parameter is
      recorded through ``saved_tensors_hooks`` (distinct storage addresses, so a tensor saved twice counts once); the
      layer's persistent basis is added when the saved basis copy is a different tensor.
    * Weight-gradient fidelity: a forward hook keeps each wrapped layer's input, a backward hook multiplies it with the
      incoming output gradient in fp32 (the dense ``dY^T X`` on the same batch and weights), and after the backward pass
      the layer's own ``weight.grad`` is compared with it by cosine.
    Returns ``{"dw_cosine_mean", "dw_cosine_worst", "dw_cosine_layers", "saved_bytes_measured", "dense_bytes"}``.
    """
    params = {p.data_ptr() for p in model.parameters()}
    state = {"inside": None, "seen": set(), "bytes": 0, "dense": 0}
    inputs, dense_dw = {}, {}

    def pack(t):
        if state["inside"] is not None and t.data_ptr() not in params and t.data_ptr() not in state["seen"]:
            state["seen"].add(t.data_ptr())
            state["bytes"] += t.numel() * t.element_size()
        return t

    def pre_hook(mod, args):
        state["inside"] = mod

    def fwd_hook(mod, args, out):
        state["inside"] = None
        x = args[0].detach()
        inputs[mod] = x
        state["dense"] += x.numel() * 2

    def bwd_hook(mod, grad_in, grad_out):
        x = inputs.pop(mod)
        dy = grad_out[0]
        x2 = x.reshape(-1, x.shape[-1]).float()
        d2 = dy.reshape(-1, dy.shape[-1]).float()
        dense_dw[mod] = d2.t() @ x2          # [out, in], fp32 (no TF32)

    handles = []
    for layer in layers:
        handles += [layer.register_forward_pre_hook(pre_hook), layer.register_forward_hook(fwd_hook),
                    layer.register_full_backward_hook(bwd_hook)]
    try:
        with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
            run_forward_backward()
        torch.cuda.synchronize()
    finally:
        for h in handles:
            h.remove()
    for layer in layers:                      # persistent bases that the saved tensors did not already cover
        basis = getattr(layer, "basis", None)
        if basis is not None and basis.data_ptr() not in state["seen"]:
            state["bytes"] += basis.numel() * basis.element_size()
    cosines = []
    for layer in layers:
        ref = dense_dw.pop(layer, None)
        grad = layer.weight.grad
        if ref is None or grad is None:
            continue
        g = grad.detach().float()
        if g.shape != ref.shape:
            g = g.t()
        denom = float(g.norm() * ref.norm())
        cosines.append(float((g * ref).sum()) / denom if denom > 0 else 1.0)
        del ref
    return {"dw_cosine_mean": sum(cosines) / max(1, len(cosines)), "dw_cosine_worst": min(cosines) if cosines else None,
            "dw_cosine_layers": len(cosines), "saved_bytes_measured": state["bytes"], "dense_bytes": state["dense"]}


PREP_STEPS = 5              # untimed training steps on batches 0..4 before the warm-up, identical in both arms (see run_ours)
EVIDENCE_STEPS = 8          # one per synthetic batch: the tracked bases favour the batches seen last, so a single batch would
                            # make the figure depend on where in the cycle the timed regions happened to stop


def guarded_evidence(torch, model, layers, run_forward_backward):
    """The evidence steps must never cost the benchmark its line: a failure is reported on stderr and the fields stay null.

    ``run_forward_backward(i)`` runs one training-mode forward + backward on synthetic batch ``i``; it is called for every batch
    of the cycle and the cosines are averaged (worst = worst layer of any batch).  Saved bytes are those of the first step."""
    try:
        runs = [fidelity_and_saved_bytes(torch, model, layers, lambda i=i: run_forward_backward(i)) for i in range(EVIDENCE_STEPS)]
        out = dict(runs[0])
        out["dw_cosine_mean"] = sum(r["dw_cosine_mean"] for r in runs) / len(runs)
        worst = [r["dw_cosine_worst"] for r in runs if r["dw_cosine_worst"] is not None]
        out["dw_cosine_worst"] = min(worst) if worst else None
        out["dw_cosine_per_batch"] = [round(r["dw_cosine_mean"], 4) for r in runs]
        return out
    except Exception as exc:  # noqa: BLE001
        print(f"evidence step failed: {type(exc).__name__}: {exc}", file=sys.stderr, flush=True)
        return None


def timed_regions(torch, dist, steps, step_fn, world, repeats):
    """``repeats`` back-to-back timed regions of ``steps`` steps; returns (median seconds, all seconds)."""
    all_secs = [timed_region(torch, dist, steps, step_fn, world) for _ in range(max(1, repeats))]
    return statistics.median(all_secs), all_secs



class LossReader:
    """Device-to-host read of every step's loss through pinned memory without idling the GPU between steps.

    The 4-byte copy of step i is queued right behind the step; the host waits for it only after step i+1 has been queued
    (``drain`` waits for the last one, inside the timed region).  Every step's loss is read; the bytes per step are unchanged.
    Both arms of the benchmark use the same reader.
    """

    def __init__(self, torch):
        self.torch = torch
        self.buf = torch.empty(2, dtype=torch.float32).pin_memory()
        self.events = [torch.cuda.Event(), torch.cuda.Event()]
        self.count, self.value = 0, None

    def push(self, loss):
        slot = self.count & 1
        self.buf[slot:slot + 1].copy_(loss.detach().float().reshape(1), non_blocking=True)
        self.events[slot].record()
        if self.count:
            self.events[slot ^ 1].synchronize()
            self.value = float(self.buf[slot ^ 1])
        self.count += 1

    def drain(self):
        if self.count:
            slot = (self.count - 1) & 1
            self.events[slot].synchronize()
            self.value = float(self.buf[slot])
        return self.value


def make_tokens(torch, vocab, batch, seq, count, seed):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (batch, seq), generator=gen) for _ in range(count)]


def emit(payload):
    print(json.dumps(payload), flush=True)


# ----------------------------------------------------------------------------------- this framework
def kernel_table(torch, step, path, steps=2):
    """Device time per kernel name over `steps` steps (torch.profiler / CUPTI), written as text.  Not part of any timed region."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(steps):
            step(i)
        torch.cuda.synchronize()
    rows = []
    for e in prof.key_averages():
        t = getattr(e, "device_time_total", None) or getattr(e, "cuda_time_total", 0)
        if t:
            rows.append((t / steps / 1e3, e.count // steps, e.key))
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    with open(path, "w") as fh:
        fh.write(f"kernel time per step: {total:.2f} ms over {sum(r[1] for r in rows)} launches\n")
        for ms, n, name in rows[:60]:
            fh.write(f"{ms:9.3f} ms {100 * ms / total:5.1f}% {n:6d}x  {name[:110]}\n")


def gap_report(torch, step, path, steps=2):
    """Where the GPU idles inside a step: kernel intervals of `steps` profiled steps are merged and every gap longer than
    20 us is listed with the host operation that was running when the gap ended.  Written as text; not part of any timed region."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        for i in range(steps):
            step(i)
        torch.cuda.synchronize()
    events = prof.events()
    kernels = sorted(((e.time_range.start, e.time_range.end, e.name) for e in events if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda t: t[0])
    host = sorted(((e.time_range.start, e.time_range.end, e.name) for e in events if e.device_type == torch.autograd.DeviceType.CPU),
                  key=lambda t: t[0])
    if not kernels:
        return
    gaps, busy_end = [], kernels[0][1]
    for start, end, name in kernels[1:]:
        if start - busy_end > 20:
            running = [h for h in host if h[0] <= start <= h[1]]
            top = max(running, key=lambda h: h[1] - h[0])[2] if running else "-"
            leaf = min(running, key=lambda h: h[1] - h[0])[2] if running else "-"
            gaps.append((start - busy_end, name[:60], top[:50], leaf[:50]))
        busy_end = max(busy_end, end)
    span = kernels[-1][1] - kernels[0][0]
    idle = sum(g[0] for g in gaps)
    by = {}
    for g in gaps:
        key = (g[2], g[3])
        by[key] = (by.get(key, (0, 0))[0] + g[0], by.get(key, (0, 0))[1] + 1)
    with open(path, "w") as fh:
        fh.write(f"span {span / 1e3 / steps:.2f} ms per step, idle in gaps > 20 us: {idle / 1e3 / steps:.2f} ms per step over {len(gaps) // steps} gaps\n")
        fh.write("idle ms/step  gaps/step  outermost host op  |  innermost host op when the next kernel started\n")
        for (top, leaf), (us, n) in sorted(by.items(), key=lambda kv: -kv[1][0])[:40]:
            fh.write(f"{us / 1e3 / steps:10.3f} {n // steps:8d}  {top}  |  {leaf}\n")
        fh.write("largest single gaps (us, next kernel, host op):\n")
        for g in sorted(gaps, reverse=True)[:25]:
            fh.write(f"{g[0]:10.0f}  {g[1]}  |  {g[3]}\n")


def run_ours(args):
    sys.path.insert(0, REPO)
    import torch
    import torch.distributed as dist

    import stacr_b200 as S
    from stacr_b200.models import GPTNeoXForCausalLM, NeoXConfig
    from stacr_b200.ops import _lib
    from stacr_b200.optim import AdamW8bit
    from stacr_b200.parallel import GradSync, ShardedGradSync, broadcast_parameters, init_distributed

    rank, world, local = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    shape = SMALL if args.small else MODEL
    seq, batch = (512, 4) if args.small else (SEQ, BATCH)
    model = GPTNeoXForCausalLM(NeoXConfig(**shape)).to(dev).train()
    broadcast_parameters(model)
    layers = S.apply_stacr(model, **STACR)
    fused = [layer.weight for layer in layers] if args.fused_dw == "on" else []
    zero = world > 1 and args.zero == "on" and not fused
    zero_error = None
    if zero:
        # optimizer sharded over the ranks: buckets are reduced to their owners only, every rank updates 1/W of the matrices
        # and its update kernel stores the new bf16 weights through the NVSwitch multicast address (no separate all-gather)
        try:
            sync = ShardedGradSync(model.parameters(), backend=args.comm)
            opt = AdamW8bit(model.parameters(), lr=2e-5, weight_decay=0.0, bf16_shadow=True, shard=sync)
        except Exception as exc:  # noqa: BLE001 - e.g. a fabric that refuses the symmetric allocations: fall back to the replicated optimizer
            zero, zero_error = False, f"{type(exc).__name__}: {str(exc)[:160]}"
            print(f"[bench] sharded optimizer unavailable on rank {rank}, using the replicated one: {zero_error}", file=sys.stderr, flush=True)
    if not zero:
        sync = GradSync(model.parameters(), backend=args.comm, fused=fused) if world > 1 else None
        opt = AdamW8bit(model.parameters(), lr=2e-5, weight_decay=0.0, bf16_shadow=True)
    host_batches = [t.pin_memory() for t in make_tokens(torch, shape["vocab_size"], batch, seq, 8, 100 + rank)]
    dev_batches = [t.to(dev) for t in host_batches]
    counter = {"step": 0}

    def core_step(ids):
        if sync is not None:
            sync.zero_grad()
        else:
            opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        if sync is not None:
            sync.finish()
        opt.step()
        return loss

    def eager_step(ids):
        S.set_step(layers, counter["step"])
        counter["step"] += 1
        return core_step(ids)

    graphed = None
    graph_launches = 0
    graph_error = None
    if args.graph == "on" and (sync is None or sync.backend == "symm"):
        # the whole step (forward, backward, optimizer) captured once and replayed: one launch per step instead of ~2000
        from stacr_b200.graphs import GraphedStep

        # PREP_STEPS untimed training steps on batches 0..4 precede the warm-up in both arms and in the eager mode: here they are
        # two eager steps (bases initialised, caches filled), the two warm-up runs of the capture and the captured step itself
        for i in range(2):
            eager_step(dev_batches[i])
        before = _lib.launch_count() + opt.kernel_launches
        try:
            graphed = GraphedStep(core_step, [dev_batches[0]], optimizer=opt, layers=layers, first_step=counter["step"], warmup=2,
                                  prep_inputs=[[dev_batches[2]], [dev_batches[3]], [dev_batches[4]]])
            counter["step"] += 3
            graph_launches = (_lib.launch_count() + opt.kernel_launches - before) // 3     # two warm-up runs and the capture
        except Exception as exc:  # noqa: BLE001 - a capture the driver refuses must not cost the measurement: time the eager step
            graphed, graph_error = None, f"{type(exc).__name__}: {str(exc)[:160]}"
            torch.cuda.synchronize()
            print(f"[bench] CUDA graph capture failed on rank {rank}, timing the eager step instead: {graph_error}", file=sys.stderr, flush=True)

    if graphed is None:
        for i in range(0 if graph_error is None else 2, PREP_STEPS):
            eager_step(dev_batches[i])

    def train_step(ids):
        if graphed is not None:
            counter["step"] += 1
            return graphed(ids)
        return eager_step(ids)

    def step_device(i):
        train_step(dev_batches[i % len(dev_batches)])

    last = {}
    reader = LossReader(torch)

    def step_e2e(i):
        ids = host_batches[i % len(host_batches)].to(dev, non_blocking=True)  # pinned host -> device
        reader.push(train_step(ids))                                            # device -> host read-back, one step behind
        if i == args.steps - 1:
            last["loss"] = reader.drain()

    warm = max(3, args.warmup)
    for i in range(warm):
        step_e2e(i)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    torch.cuda.reset_peak_memory_stats(dev)
    launches0 = _lib.launch_count() + opt.kernel_launches
    with ClockSampler(local) as clocks:
        secs, secs_all = timed_regions(torch, dist, args.steps, step_device, world, args.repeats)
    launches = (_lib.launch_count() + opt.kernel_launches - launches0) // max(1, args.repeats)
    if graphed is not None:
        launches = graph_launches * args.steps          # the kernels inside the graph, replayed once per step
    with ClockSampler(local) as clocks_e2e:
        secs_e2e, secs_e2e_all = timed_regions(torch, dist, args.steps, step_e2e, world, args.repeats)
    _lib.check_status(dev)
    peak = torch.cuda.max_memory_allocated(dev)

    def evidence_step(i):
        S.set_step(layers, counter["step"] + 8)
        counter["step"] += 1
        if sync is not None:
            sync.zero_grad()
        else:
            opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(input_ids=dev_batches[i % len(dev_batches)], labels=dev_batches[i % len(dev_batches)]).loss
        if sync is not None:
            with sync.no_sync():            # the rank's own gradient is what is compared with its own dense dY^T X: no reduction
                loss.backward()
        else:
            loss.backward()

    evidence = None if args.no_evidence else guarded_evidence(torch, model, layers, evidence_step)
    if args.kernel_table:  # every rank runs the extra steps (their collectives need all ranks); rank 0 writes the table
        kernel_table(torch, step_device, args.kernel_table if rank == 0 else os.devnull)
    if args.gap_report:
        gap_report(torch, step_device, args.gap_report if rank == 0 else os.devnull)
    rows = batch * seq
    factor_bytes = sum(layer.stored_bytes(rows, 2)["total"] for layer in layers)
    dense_bytes = sum(rows * layer.in_features * 2 for layer in layers)
    tokens = world * batch * seq * args.steps
    if rank == 0:
        emit({
            "metric": "tokens_per_second", "value": tokens / secs, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights", "impl": "stacr_b200",
            "config": {
                "model": "pythia-1.4b-shaped (24L d2048 h16 mlp8192 rotary25% parallel-residual vocab50304)" if not args.small else "small",
                "global_batch": world * batch, "seq_len": seq, "parallelism": f"dp{world}",
                "stacr": STACR, "optimizer": "AdamW 8-bit block-wise (in-tree)", "comm": sync.backend if sync else "none",
                "fused_dw_reduce_scatter": bool(sync and sync.n_fused and sync.backend == "symm"),
                "optimizer_sharding": "ZeRO-1: reduce-to-owner buckets, 1/W optimizer per rank, bf16 weights published by multicast stores of the update kernel" if zero else "replicated",
                "l2": "inputs larger than L2: every step streams 2.8 GB of bf16 weights and > 10 GB of activations through a 126 MB L2",
                "cuda_graph": graphed is not None,
                **({"cuda_graph_error": graph_error} if graph_error else {}),
                **({"optimizer_sharding_error": zero_error} if zero_error else {}),
                "attention": "in-tree tcgen05 forward + backward on the fused QKV projection" if args.attention == "intree" else "library (scaled_dot_product_attention)",
            },
            "clocks": clocks.summary(),
            "timing": {"regions": len(secs_all), "steps_per_region": args.steps, "reported": "median region",
                       "ms_per_step_regions": [1e3 * t / args.steps for t in secs_all],
                       "e2e_ms_per_step_regions": [1e3 * t / args.steps for t in secs_e2e_all]},
            "e2e": {"value": tokens / secs_e2e, "unit": "tokens/s", "h2d_bytes_per_step": batch * seq * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": 1e3 * secs_e2e / args.steps, "last_loss": last.get("loss"), "clocks": clocks_e2e.summary(),
                    "how": "own timed region: per step a pinned-host token batch is copied to the device and the loss is copied back to pinned memory and read by the host one step later (the last one inside the region)"},
            "gpu_launches": launches,
            "memory": {"peak_allocated_gb": peak / 1e9, "saved_activation_gb_wrapped_layers": factor_bytes / 1e9,
                       "dense_saved_gb_same_layers": dense_bytes / 1e9,
                       "saved_activation_gb_wrapped_layers_measured": None if evidence is None else evidence["saved_bytes_measured"] / 1e9,
                       "how": "measured: bytes of the non-parameter tensors autograd saved inside the wrapped layers' forwards (saved_tensors_hooks) plus their persistent bases; the unsuffixed figure is the layers' stored_bytes() formula"},
            "fidelity": None if evidence is None else {
                "dw_cosine_mean": evidence["dw_cosine_mean"], "dw_cosine_worst": evidence["dw_cosine_worst"], "layers": evidence["dw_cosine_layers"],
                "dw_cosine_per_batch": evidence.get("dw_cosine_per_batch"),
                "how": "eight extra forward + backward passes after the timed regions, one per synthetic batch, no optimizer step: each wrapped layer's weight.grad against fp32 dY^T X formed from the same input and output gradient; mean over layers and batches, worst layer of any batch"},
        })
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------- reference
def run_reference(args):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "stacr")):
        emit({"impl": "reference", "unavailable": "baseline/_ref is missing (offline pip install of the reference not present)"})
        return
    # The reference package is also called `stacr`: keep this repository off the import path.
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != REPO]
    sys.path.insert(0, ref_root)
    try:
        import torch
        import torch.distributed as dist
        import stacr as ref
        from torch.nn.parallel import DistributedDataParallel as DDP
        from transformers import GPTNeoXConfig, GPTNeoXForCausalLM
    except Exception as exc:  # noqa: BLE001
        emit({"impl": "reference", "unavailable": f"import failed: {type(exc).__name__}: {exc}"[:300]})
        return
    assert os.path.abspath(ref.__file__).startswith(ref_root), ref.__file__
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(1234)
    shape = SMALL if args.small else MODEL
    seq, batch = (512, 4) if args.small else (SEQ, BATCH)
    model = GPTNeoXForCausalLM(GPTNeoXConfig(**shape, hidden_dropout=0.0, attention_dropout=0.0)).to(dev).train()
    layers = ref.apply_stacr(model, **STACR)
    net = DDP(model, device_ids=[local], static_graph=True, broadcast_buffers=False) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=2e-5, weight_decay=0.0)
    host_batches = [t.pin_memory() for t in make_tokens(torch, shape["vocab_size"], batch, seq, 8, 100 + rank)]
    dev_batches = [t.to(dev) for t in host_batches]
    counter = {"step": 0}

    def train_step(ids):
        ref.set_step(layers, counter["step"])
        counter["step"] += 1
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(input_ids=ids, labels=ids).loss
        loss.backward()
        opt.step()
        return loss

    last = {}

    def step_device(i):
        train_step(dev_batches[i % len(dev_batches)])

    reader = LossReader(torch)

    def step_e2e(i):
        ids = host_batches[i % len(host_batches)].to(dev, non_blocking=True)
        reader.push(train_step(ids))
        if i == args.steps - 1:
            last["loss"] = reader.drain()

    for i in range(PREP_STEPS):                 # the same untimed steps on batches 0..4 that this framework's arm takes
        step_device(i)
    warm = max(3, args.warmup)
    for i in range(warm):
        step_e2e(i)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats(dev)
    with ClockSampler(local) as clocks:
        secs, secs_all = timed_regions(torch, dist, args.steps, step_device, world, args.repeats)
    with ClockSampler(local) as clocks_e2e:
        secs_e2e, secs_e2e_all = timed_regions(torch, dist, args.steps, step_e2e, world, args.repeats)
    peak = torch.cuda.max_memory_allocated(dev)

    def evidence_step(i):
        ref.set_step(layers, counter["step"])
        counter["step"] += 1
        opt.zero_grad(set_to_none=True)
        # under DDP the pass runs without the gradient all-reduce: a rank's own gradient is compared with its own dense dY^T X
        with (net.no_sync() if world > 1 else contextlib.nullcontext()):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = net(input_ids=dev_batches[i % len(dev_batches)], labels=dev_batches[i % len(dev_batches)]).loss
            loss.backward()

    evidence = None if args.no_evidence else guarded_evidence(torch, model, layers, evidence_step)
    rows = batch * seq
    factor_bytes = sum(layer.stored_bytes(rows, 2)["total"] for layer in layers)
    tokens = world * batch * seq * args.steps
    if rank == 0:
        emit({
            "impl": "reference", "metric": "tokens_per_second", "value": tokens / secs, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": 1e3 * secs / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {
                "model": "pythia-1.4b-shaped (HF GPTNeoXForCausalLM from config)" if not args.small else "small",
                "global_batch": world * batch, "seq_len": seq, "parallelism": f"dp{world}", "stacr": STACR,
                "optimizer": "torch.optim.AdamW (the reference's 8-bit optimizer needs bitsandbytes, not installed)",
                "ddp": "torch DistributedDataParallel(static_graph=True, broadcast_buffers=False)",
                "l2": "inputs larger than L2",
            },
            "clocks": clocks.summary(),
            "e2e": {"value": tokens / secs_e2e, "unit": "tokens/s", "h2d_bytes_per_step": batch * seq * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": 1e3 * secs_e2e / args.steps, "last_loss": last.get("loss"), "clocks": clocks_e2e.summary(),
                    "how": "own timed region: per step a pinned-host token batch is copied to the device and the loss is copied back to pinned memory and read by the host one step later (the last one inside the region)"},
            "gpu_launches": None,
            "timing": {"regions": len(secs_all), "steps_per_region": args.steps, "reported": "median region",
                       "ms_per_step_regions": [1e3 * t / args.steps for t in secs_all],
                       "e2e_ms_per_step_regions": [1e3 * t / args.steps for t in secs_e2e_all]},
            "memory": {"peak_allocated_gb": peak / 1e9, "saved_activation_gb_wrapped_layers": factor_bytes / 1e9,
                       "saved_activation_gb_wrapped_layers_measured": None if evidence is None else evidence["saved_bytes_measured"] / 1e9,
                       "dense_saved_gb_same_layers": None if evidence is None else evidence["dense_bytes"] / 1e9},
            "fidelity": None if evidence is None else {
                "dw_cosine_mean": evidence["dw_cosine_mean"], "dw_cosine_worst": evidence["dw_cosine_worst"], "layers": evidence["dw_cosine_layers"],
                "dw_cosine_per_batch": evidence.get("dw_cosine_per_batch"),
                "how": "eight extra forward + backward passes after the timed regions, one per synthetic batch, no optimizer step: each wrapped layer's weight.grad against fp32 dY^T X formed from the same input and output gradient; mean over layers and batches, worst layer of any batch"},
        })
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--comm", default="auto", choices=["auto", "symm", "nccl"], help="gradient all-reduce path (this framework)")
    ap.add_argument("--fused-dw", default="off", choices=["on", "off"],
                    help="N > 1: compressed layers' weight-gradient kernels reduce-scatter in their epilogue over NVLink peer memory")
    ap.add_argument("--graph", default="on", choices=["on", "off"],
                    help="capture the training step (with the in-tree collectives at N > 1) into a CUDA graph and replay it")
    ap.add_argument("--zero", default="on", choices=["on", "off"], help="N > 1: shard the optimizer over the ranks (reduce-to-owner + multicast weight publication)")
    ap.add_argument("--attention", default="library", choices=["library", "intree"],
                    help="softmax attention: the fused library kernel (default, faster) or the in-tree tcgen05 forward + backward")
    ap.add_argument("--gap-report", metavar="FILE", help="after the timed regions, write where the GPU idles inside two more steps to FILE")
    ap.add_argument("--kernel-table", metavar="FILE", help="after the timed regions, write per-kernel device times of two more steps to FILE")
    ap.add_argument("--small", action="store_true", help="tiny shape for smoke runs (not a benchmark number)")
    ap.add_argument("--repeats", type=int, default=3, help="timed regions of --steps steps per measurement; the median region is reported")
    ap.add_argument("--no-evidence", action="store_true", help="skip the extra step that measures dW cosine and saved bytes after the timed regions")
    args = ap.parse_args()
    if args.impl == "ours":
        os.environ["STACR_ATTENTION"] = args.attention
    if args.gpus > 1 and "RANK" not in os.environ:
        raise SystemExit("for --gpus > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    (run_reference if args.impl == "reference" else run_ours)(args)


if __name__ == "__main__":
    main()
