"""Shared machinery of the measurement grids: one matched training cell, paired gradient fidelity, SSP ledger, JSONL output.

``run_config`` runs one cell: build the model (in-tree random init when weights are not available offline), apply
selective checkpointing / CPU offload / freezing / STAC-R on chosen blocks, pre-stage all batches on the device,
train with the device-timed loop, and return peak memory, tokens/s, losses and validation perplexity.
Parity: experiments/benchmarks/common.py:22-686 of the reference project.  Timing uses CUDA events instead of a
host clock.
"""

from __future__ import annotations

import gc
import json
import math
import os
import time
import uuid
from contextlib import nullcontext
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Optional

import torch

import stacr_b200 as S
from stacr_b200.composition import block_target_names, checkpoint_blocks, offload_blocks, transformer_blocks
from stacr_b200.models import build_model, load_model_and_tokenizer
from stacr_b200.utils import set_seed  # noqa: F401  (re-exported for the grids)

RESULTS = Path(os.environ.get("STACR_RESULTS", "results"))
RUN_ID = os.environ.get("STACR_RUN_ID") or uuid.uuid4().hex[:12]
QUIET = os.environ.get("STACR_QUIET", "0") == "1"
PARAMETERS: Dict[str, Any] = {}
_RECORDER: Optional[Callable[..., dict]] = None  # set by the dry-run planner: cells are recorded, not run


def configure(**overrides) -> None:
    """Install CLI overrides (steps, model_id, bs, seq, ...) that ``resolve_parameters`` merges into grid defaults."""
    PARAMETERS.clear()
    PARAMETERS.update({k: v for k, v in overrides.items() if v is not None})
    if "STACR_STEPS" in os.environ and "steps" not in PARAMETERS:
        PARAMETERS["steps"] = int(os.environ["STACR_STEPS"])


def resolve_parameters(**defaults) -> Dict[str, Any]:
    return {**defaults, **{k: v for k, v in PARAMETERS.items() if k in defaults or k in ("device", "optimizer", "dataset", "attn_impl")}}


def set_recorder(fn: Optional[Callable[..., dict]]) -> None:
    global _RECORDER
    _RECORDER = fn


def sync() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def free_all() -> None:
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()


def gib(n: float) -> float:
    return n / 1024**3


def amp_ctx(enabled: bool = True, dtype=torch.bfloat16):
    if not enabled:
        return nullcontext()
    return torch.autocast("cuda" if torch.cuda.is_available() else "cpu", dtype=dtype)


def load_model(model_id: str, device: str = "cuda", dtype=torch.float32, attn_impl: Optional[str] = None, **overrides):
    """In-tree architecture by preset name when known (random init), else Hugging Face weights from the local cache."""
    try:
        model = build_model(model_id, **overrides)
    except KeyError:
        model, _ = load_model_and_tokenizer(model_id, dtype=dtype, attn_implementation=attn_impl, local_files_only=True)
    return model.to(device=device, dtype=dtype).train()


def get_batches(model_id: str, split: str, bs: int, seq: int, count: int, dataset: str = "synthetic", device: str = "cuda", vocab: Optional[int] = None, seed: int = 0,
                num_labels: int = 0):
    """``count`` batches resident on ``device`` (uniform-random tokens offline): language-model labels, or with ``num_labels``
    one random class per sequence (a memory/throughput protocol; quality columns of such rows are not meaningful)."""
    gen = torch.Generator().manual_seed(seed + (1 if split != "train" else 0))
    vocab = vocab or 50257
    out = []
    for _ in range(count):
        ids = torch.randint(0, vocab, (bs, seq), generator=gen).to(device)
        labels = torch.randint(0, num_labels, (bs,), generator=gen).to(device) if num_labels else ids.clone()
        out.append({"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": labels})
    return out


def build_optimizer(model, lr: float = 5e-5, eight_bit: bool = True, weight_decay: float = 0.0, kind: Optional[str] = None):
    """AdamW (8-bit block-wise by default on CUDA); ``kind`` ``"subtrack"``/``"galore"`` builds the low-rank-state optimizers."""
    from stacr_b200.optim import AdamW, AdamW8bit

    if kind in ("subtrack", "galore"):
        from stacr_b200.comparators.galore_adapter import create_galore_optimizer
        from stacr_b200.comparators.subtrack_adapter import create_subtrack_optimizer

        if kind == "subtrack":
            return create_subtrack_optimizer(model, {"lr": lr, "weight_decay": weight_decay})
        return create_galore_optimizer(model, lr=lr, rank=8, weight_decay=weight_decay)
    params = [p for p in model.parameters() if p.requires_grad]
    name = kind or PARAMETERS.get("optimizer", "adamw8bit" if eight_bit else "adamw")
    if name == "adamw8bit" and params and params[0].is_cuda:
        return AdamW8bit(params, lr=lr, weight_decay=weight_decay)
    if params and params[0].is_cuda:
        return AdamW(params, lr=lr, weight_decay=weight_decay)
    return torch.optim.AdamW(params, lr=lr, weight_decay=weight_decay)


def apply_selective_checkpointing(model, every: int, offset: int = 0) -> int:
    if not every:
        return 0
    blocks = transformer_blocks(model)
    return len(checkpoint_blocks(blocks, [i for i in range(len(blocks)) if i % every == offset]))


def apply_selective_offload(model, every: int, offset: int = 0) -> int:
    if not every:
        return 0
    blocks = transformer_blocks(model)
    return len(offload_blocks(blocks, [i for i in range(len(blocks)) if i % every == offset]))


def stacr_on_blocks(model, cfg: dict, block_pred: Optional[Callable[[int], bool]] = None):
    """Apply STAC-R, optionally only to projections inside blocks selected by ``block_pred(index)``."""
    cfg = dict(cfg)
    cfg.setdefault("turbo_after_step", None)
    if block_pred is None:
        return S.apply_stacr(model, **cfg)
    blocks = transformer_blocks(model)
    sel = {k: cfg.pop(k) for k in list(cfg) if k in ("surface", "min_features", "extra_names", "exclude_names", "trainable_only")}
    names = block_target_names(model, blocks, block_pred, **sel)
    return S.apply_stacr(model, surface="none", target_names=names, allow_empty=True, **cfg)


def runtime_metadata() -> dict:
    """Versions of the libraries in use, the CUDA toolkit torch was built for, the device name and whether the
    in-tree kernel library is loaded.  Environment variables are never recorded."""
    import importlib.metadata as md

    versions = {}
    for name in ("torch", "transformers", "datasets", "numpy"):
        try:
            versions[name] = md.version(name)
        except md.PackageNotFoundError:
            pass
    from stacr_b200.ops import _lib

    return {"versions": versions, "cuda": torch.version.cuda, "device": torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu",
            "kernel_library": bool(_lib.available())}


def nvml_used(dev: int = 0) -> float:
    """Device memory in use according to NVML, in GiB (all processes); NaN without NVML.  Read-only query."""
    try:
        import pynvml

        pynvml.nvmlInit()
        return gib(pynvml.nvmlDeviceGetMemoryInfo(pynvml.nvmlDeviceGetHandleByIndex(dev)).used)
    except Exception:
        return float("nan")


def blocks_of(model) -> list:
    """The model's transformer blocks (``RuntimeError`` for an unknown layout)."""
    try:
        return transformer_blocks(model)
    except ValueError as exc:
        raise RuntimeError(f"cannot locate blocks for {type(model).__name__}") from exc


def apply_cpu_offload(model, every: int = 1, offset: int = 0) -> int:
    """Keep the saved tensors of every ``every``-th block in pinned host memory; returns the number of blocks."""
    return apply_selective_offload(model, every, offset)


def freeze_surface_params(model, surface: str = "mlp", min_features: int = 256) -> int:
    """Turn off gradients of the projections a surface selects (for probes that train everything else); returns the count."""
    names = set(S.select_target_names(model, surface=surface, min_features=min_features))
    count = 0
    for name, module in model.named_modules():
        if name in names:
            for p in module.parameters(recurse=False):
                p.requires_grad_(False)
                count += 1
    return count


def restrict_cfg_to_blocks(model, cfg: dict, block_pred: Callable[[int], bool]) -> dict:
    """A copy of ``cfg`` whose selection is the explicit list of surface projections inside the chosen blocks."""
    names = block_target_names(model, transformer_blocks(model), block_pred, surface=str(cfg.get("surface", "mlp")),
                               min_features=int(cfg.get("min_features", 256)))
    out = dict(cfg)
    out["surface"], out["extra_names"] = "none", names
    return out


def instrument_rows(layers) -> tuple:
    """Count the rows (tokens) each layer sees: ``(rows_by_module_id, hook_handles)``; remove the handles when done."""
    rows: Dict[int, int] = {}

    def count(module, inputs):
        x = inputs[0]
        rows[id(module)] = rows.get(id(module), 0) + x.numel() // x.shape[-1]

    return rows, [layer.register_forward_pre_hook(count) for layer in layers]


@torch.no_grad()
def validation_ppl(model, batches, amp: bool = True) -> float:
    """Token-weighted perplexity over ``batches`` (each sequence contributes ``len - 1`` predictions)."""
    was_training = model.training
    model.eval()
    nll, count = 0.0, 0
    for batch in batches:
        with amp_ctx(amp and batch["input_ids"].is_cuda):
            loss = model(**batch).loss
        n = batch["labels"].numel() - batch["labels"].shape[0]
        nll += float(loss) * n
        count += n
    model.train(was_training)
    return math.exp(min(nll / max(count, 1), 50.0))


class SSPLedger:
    """Saved-surface predictor inputs: bytes autograd would save densely for the wrapped layers vs factor bytes."""

    def __init__(self, layers, value_bytes: int = 2):
        self.layers, self.value_bytes = list(layers), value_bytes
        self.wrapped_bytes = self.payload_bytes = self.basis_bytes = 0
        self.probed = False

    def probe(self, rows: int) -> None:
        if self.probed:
            return
        for layer in self.layers:
            rep = layer.stored_bytes(rows, self.value_bytes)
            self.wrapped_bytes += rows * layer.in_features * self.value_bytes
            self.payload_bytes += rep["coeff"] + rep["residual"] + rep["saved_basis_cast"]
            self.basis_bytes += rep["persistent_basis"]
        self.probed = True

    def report(self, baseline_peak_bytes: Optional[int]) -> dict:
        from stacr_b200.analysis import surface_ledger

        if not self.probed or not baseline_peak_bytes:
            return {}
        return surface_ledger(self.wrapped_bytes, self.payload_bytes, baseline_peak_bytes, basis_bytes=self.basis_bytes)


def run_config(method: str, seed: int = 42, *, model_id: str = "gpt2-medium", bs: int = 8, seq: int = 1024, steps: int = 60,
               measure_from: int = 20, stacr_cfg: Optional[dict] = None, stacr_block_pred=None, ckpt_every: int = 0, ckpt_offset: int = 0,
               offload_every: int = 0, freeze_mlp: bool = False, eight_bit: bool = True, lr: float = 5e-5, amp: bool = True,
               model_dtype=torch.float32, device: Optional[str] = None, eval_batches: int = 4, dataset: str = "synthetic",
               attn_impl: Optional[str] = None, baseline_peak_bytes: Optional[int] = None, model_overrides: Optional[dict] = None, **extra) -> dict:
    """One measurement cell.  Under the dry-run planner the arguments are recorded and a placeholder row returned."""
    args = dict(method=method, seed=seed, model_id=model_id, bs=bs, seq=seq, steps=steps, measure_from=measure_from, stacr_cfg=stacr_cfg,
                ckpt_every=ckpt_every, offload_every=offload_every, freeze_mlp=freeze_mlp, eight_bit=eight_bit, dataset=dataset, **extra)
    if _RECORDER is not None:
        return _RECORDER(**args)
    device = device or PARAMETERS.get("device") or ("cuda" if torch.cuda.is_available() else "cpu")
    cuda = device == "cuda"
    free_all()
    set_seed(seed)
    model = load_model(model_id, device, dtype=model_dtype, attn_impl=attn_impl, **(model_overrides or {}))
    num_labels = int(getattr(model.config, "num_labels", 2)) if type(model).__name__.endswith("ForSequenceClassification") else 0
    adapter_report = None
    if extra.get("lora") or extra.get("qlora"):
        from stacr_b200.protocols.lora import apply_lora, trainable_parameter_report

        adapters = apply_lora(model, r=8, alpha=16.0, quantize_base=bool(extra.get("qlora")))
        adapter_report = {"adapter_rank": 8, "n_adapters": len(adapters), **trainable_parameter_report(model)}
        if stacr_cfg:                      # only trainable projections save inputs: an adapter-only run has an empty MLP surface
            stacr_cfg = dict(stacr_cfg, allow_empty=True, trainable_only=True)
            adapter_report["n_eligible_mlp_layers"] = len(S.select_target_names(model, surface=stacr_cfg.get("surface", "mlp"), min_features=int(stacr_cfg.get("min_features", 256))))
            adapter_report["empty_compression_control"] = adapter_report["n_eligible_mlp_layers"] == 0
    n_ckpt = apply_selective_checkpointing(model, ckpt_every, ckpt_offset)
    n_off = apply_selective_offload(model, offload_every, 1 if offload_every > 1 else 0)
    if freeze_mlp:
        for name in S.select_target_names(model, surface="mlp"):
            model.get_submodule(name).requires_grad_(False)
    if stacr_cfg and extra.get("basis_comparator"):
        from stacr_b200.comparators.activation import apply_comparator

        layers = apply_comparator(model, extra["basis_comparator"], dict(stacr_cfg))
    else:
        layers = stacr_on_blocks(model, stacr_cfg, stacr_block_pred) if stacr_cfg else []
    opt = build_optimizer(model, lr, eight_bit and cuda, kind=extra.get("optimizer"))
    vocab = getattr(getattr(model, "config", None), "vocab_size", None)
    train = get_batches(model_id, "train", bs, seq, steps, dataset, device, vocab, seed, num_labels)
    ledger = SSPLedger(layers)
    losses = []
    ev0 = ev1 = None
    t0 = None
    trace_at = {s_ for s_ in (10, 50, 100, 200, 300, 400, 500, steps - 1) if s_ < steps} if extra.get("trace_memory") else set()
    marks, phases = [], None
    for i, batch in enumerate(train):
        if extra.get("phase_profile") and cuda and i == min(measure_from + 1, steps - 1):
            phases = _phase_peaks(model, opt, batch, amp)
            losses.append(phases.pop("loss"))
            continue
        S.set_step(layers, i)
        if i == measure_from:
            sync()
            if cuda:
                torch.cuda.reset_peak_memory_stats()
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            t0 = time.perf_counter()
        opt.zero_grad(set_to_none=True)
        with amp_ctx(amp and cuda):
            loss = model(**batch).loss
        value = float(loss.detach())
        if not math.isfinite(value):
            raise FloatingPointError(f"Nonfinite loss at step {i}")
        loss.backward()
        opt.step()
        losses.append(value)
        ledger.probe(bs * seq)
        if i in trace_at:
            sync()
            marks.append({"step": i, "allocated_GiB": gib(torch.cuda.max_memory_allocated()) if cuda else 0.0,
                          "reserved_GiB": gib(torch.cuda.max_memory_reserved()) if cuda else 0.0, "nvml_GiB": nvml_used(0) if cuda else float("nan"),
                          "elapsed_s": time.perf_counter() - (t0 or time.perf_counter())})
    if cuda and ev0 is not None:
        ev1.record()
        sync()
        elapsed = ev0.elapsed_time(ev1) / 1e3
    else:
        elapsed = time.perf_counter() - (t0 or time.perf_counter())
    peak = torch.cuda.max_memory_allocated() if cuda else 0
    measured = max(0, steps - measure_from)
    val_ppl = None
    if eval_batches:
        model.eval()
        with torch.no_grad(), amp_ctx(amp and cuda):
            nll = [float(model(**b).loss) for b in get_batches(model_id, "validation", bs, seq, eval_batches, dataset, device, vocab, seed, num_labels)]
        val_ppl = math.exp(min(700.0, sum(nll) / len(nll)))
    row = {
        "method": method, "seed": seed, "model": model_id, "bs": bs, "seq": seq, "steps": steps, "steps_measured": measured,
        "n_checkpointed_blocks": n_ckpt, "n_offloaded_blocks": n_off, "n_wrapped_layers": len(layers), "time_s": elapsed,
        "peak_bytes": peak, "peak_GiB": gib(peak), "tokens_per_s": bs * seq * measured / elapsed if elapsed > 0 and measured else None,
        "final_train_loss": losses[-1] if losses else None, "validation_ppl": val_ppl, "data": dataset, "status": "ok",
        "ssp": ledger.report(baseline_peak_bytes), **{k: v for k, v in extra.items() if isinstance(v, (int, float, str, bool, type(None)))},
    }
    if num_labels:
        row.update(label_protocol="random_classes", quality_metric_valid=False)
    if adapter_report:
        row.update(adapter_report)
    if marks:
        row.update(marks=marks, final_allocated_GiB=marks[-1]["allocated_GiB"], final_reserved_GiB=marks[-1]["reserved_GiB"], final_nvml_GiB=marks[-1]["nvml_GiB"])
    if phases:
        row["phase_peaks_GiB"] = phases
    del model, opt, train, layers
    free_all()
    return row


def _phase_peaks(model, opt, batch, amp: bool) -> dict:
    """One training step with the allocator's peak read after each phase: where in the step the memory peak is set.

    Returns GiB figures: resident bytes before the step, the peak reached during forward, backward and the optimizer
    step, and what is still held when forward ends (the saved activations plus the loss graph).
    """
    sync()
    before = torch.cuda.memory_allocated()
    out = {"resident_before_step": gib(before)}
    opt.zero_grad(set_to_none=True)
    torch.cuda.reset_peak_memory_stats()
    with amp_ctx(amp):
        loss = model(**batch).loss
    sync()
    out["forward_peak"], out["held_after_forward"] = gib(torch.cuda.max_memory_allocated()), gib(torch.cuda.memory_allocated() - before)
    torch.cuda.reset_peak_memory_stats()
    loss.backward()
    sync()
    out["backward_peak"] = gib(torch.cuda.max_memory_allocated())
    torch.cuda.reset_peak_memory_stats()
    opt.step()
    sync()
    out["optimizer_peak"] = gib(torch.cuda.max_memory_allocated())
    out["peak_phase"] = max(("forward_peak", "backward_peak", "optimizer_peak"), key=lambda k: out[k])
    out["loss"] = float(loss.detach())
    return out


def emit(record: dict, path: str | Path) -> None:
    """Append one enriched JSON line (run id, library versions, CLI overrides)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    enriched = {"run_id": RUN_ID, "torch": torch.__version__, "stacr_b200": S.__version__, "overrides": dict(PARAMETERS),
                "hwtag": os.environ.get("STACR_HWTAG"), **record}
    with path.open("a", encoding="utf-8") as fh:
        fh.write(json.dumps(enriched, default=str) + "\n")
    if not QUIET:
        keys = ("method", "model", "peak_GiB", "tokens_per_s", "validation_ppl", "status")
        print("  " + "  ".join(f"{k}={record[k]:.4g}" if isinstance(record.get(k), float) else f"{k}={record.get(k)}" for k in keys if k in record), flush=True)


def gradient_fidelity(model_id: str, stacr_cfg: dict, *, bs: int = 2, seq: int = 256, steps: int = 6, seed: int = 42, device: Optional[str] = None,
                      model_overrides: Optional[dict] = None) -> dict:
    """Two-model paired protocol: same weights and batch, exact vs compressed gradients, cosine per step."""
    import copy

    from stacr_b200.diagnostics import compression_diagnostics

    if _RECORDER is not None:
        return _RECORDER(method="fidelity", model_id=model_id, stacr_cfg=stacr_cfg, bs=bs, seq=seq, steps=steps, seed=seed)
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    set_seed(seed)
    ref = load_model(model_id, device, **(model_overrides or {}))
    test = copy.deepcopy(ref)
    paired = dict(test.named_parameters())
    layers = stacr_on_blocks(test, stacr_cfg)
    wrapped = {l.source_name + ".weight" for l in layers}
    vocab = getattr(getattr(ref, "config", None), "vocab_size", None)
    batches = get_batches(model_id, "train", bs, seq, steps, "synthetic", device, vocab, seed)
    whole, local = [], []
    for step, batch in enumerate(batches):
        S.set_step(layers, step)
        with torch.no_grad():
            pass
        test.train()
        with amp_ctx(device == "cuda"):
            test(**batch)  # fits / refreshes the bases
        for m in (ref, test):
            m.zero_grad(set_to_none=True)
            with compression_diagnostics(m), amp_ctx(device == "cuda"):
                m(**batch).loss.backward()
        dot = na = nb = 0.0
        for name, p in ref.named_parameters():
            if p.grad is None or paired[name].grad is None:
                continue
            a, b = p.grad.double(), paired[name].grad.double()
            d, x, y = float((a * b).sum()), float(a.square().sum()), float(b.square().sum())
            dot, na, nb = dot + d, na + x, nb + y
            if name in wrapped and x * y > 0:
                local.append(d / math.sqrt(x * y))
        whole.append(dot / math.sqrt(na * nb) if na * nb > 0 else 1.0)
    return {"model": model_id, "steps": steps, "mean_cosine": sum(whole) / len(whole), "worst_cosine": min(whole),
            "local_mean_cosine": sum(local) / len(local) if local else None, "local_worst_cosine": min(local) if local else None,
            "wrapped_layers": len(layers)}
