"""Stand-alone pieces of the convergence protocol: memory readouts, data and model factories, target lists,
storage estimators and a one-epoch loop.

``run_convergence_experiment`` composes the same steps inline; these functions expose them one by one for scripts
that build their own run (parity: experiments/protocols/training.py:371-416 memory readouts, :494-510 DDP helpers,
:531-795 data/model factories, :796-884 target lists and reshape shapes, :1014-1036 min-adaptation rule,
:1562-1975 storage estimators, :2038-2045 ``BaselineState``, :3484-4030 ``train_epoch``).  Every name is
re-exported by ``experiments.protocols.training``.
"""

from __future__ import annotations

import math
import time
import warnings
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn

from stacr_b200 import memory_accounting as acct
from stacr_b200.protocols.profiling import read_peaks

__all__ = [
    "measure_memory_for_cap", "measure_memory_for_report", "log_memory_complete", "cleanup_ddp", "wrap_model_ddp",
    "setup_sst2_data", "create_bert_sst2", "setup_wikitext_data", "create_gpt2_lm", "get_compression_targets_gpt2",
    "get_compression_targets_bert", "auto_reshape_shape", "apply_min_adaptation_rule", "estimate_storage_for_model",
    "estimate_storage_for_stacr", "estimate_storage_for_c1", "estimate_storage_for_prac", "BaselineState", "train_epoch",
]


# ------------------------------------------------------------------------------ memory readouts
def _peak(field: str) -> Optional[int]:
    peaks = read_peaks()
    return peaks.get(field) if peaks.get("device_mode") == "cuda" else None


def measure_memory_for_cap() -> Optional[int]:
    """Peak *reserved* bytes: the conservative figure used when calibrating runs to an equal memory cap."""
    return _peak("max_reserved_bytes")


def measure_memory_for_report() -> Optional[int]:
    """Peak *allocated* bytes: the figure reported in tables."""
    return _peak("max_allocated_bytes")


def log_memory_complete(logger: Any, step: int) -> Dict[str, Any]:
    """Write both peaks (and the allocator's overhead in per cent of allocated) to the run's profile log."""
    peaks = read_peaks()
    alloc, reserved = peaks.get("max_allocated_bytes"), peaks.get("max_reserved_bytes")
    info: Dict[str, Any] = {"step": step, "device_mode": peaks.get("device_mode"), "peak_allocated_bytes": alloc,
                            "peak_reserved_bytes": reserved}
    if isinstance(alloc, (int, float)) and isinstance(reserved, (int, float)) and alloc > 0:
        info["allocator_overhead_pct"] = 100.0 * max(0, reserved - alloc) / alloc
    if hasattr(logger, "log_profile"):
        logger.log_profile(info)
    return info


# ------------------------------------------------------------------------------ data parallel
def cleanup_ddp() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


def wrap_model_ddp(model: nn.Module, local_rank: int, bucket_mb: float = 25.0):
    """Synchronise the replicas' parameters and return ``(model, GradSync)``.

    Gradients live in one flat buffer reduced bucket by bucket while backward runs; saved-activation factors and
    bases stay rank-local.  The caller runs ``sync.zero_grad()`` before and ``sync.finish()`` after each backward.
    """
    from stacr_b200.parallel import GradSync, broadcast_parameters

    broadcast_parameters(model)
    return model, GradSync(model.parameters(), bucket_mb=bucket_mb)


# ------------------------------------------------------------------------------ data and models
def _loaders(cfg, vocab: int, task: str):
    from stacr_b200.datasets import build_examples, synthetic_token_examples

    def batched(examples):
        bs = int(cfg.batch_size)
        keys = examples[0].keys()
        return [{k: torch.stack([torch.as_tensor(e[k]) for e in examples[i:i + bs]]) for k in keys}
                for i in range(0, len(examples) - bs + 1, bs)] or [{k: torch.stack([torch.as_tensor(e[k]) for e in examples]) for k in keys}]

    kind = "sequence_classification" if task == "sst2" else "language_modeling"
    n_train, n_val = int(getattr(cfg, "train_examples", 64)), int(getattr(cfg, "eval_examples", 32))
    tokenizer = None
    if not getattr(cfg, "synthetic_data", True):
        try:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(cfg.model or ("bert-base-uncased" if task == "sst2" else "gpt2"), local_files_only=True)
            spec = {"dataset": "glue/sst2" if task == "sst2" else "wikitext103", "seq_len": cfg.max_length, "task": kind,
                    "train_examples": n_train, "eval_examples": n_val, "seed": cfg.seed}
            return batched(build_examples(spec, tokenizer)), batched(build_examples(spec, tokenizer, validation=True)), tokenizer
        except Exception:
            tokenizer = None
    train = synthetic_token_examples(n_train, cfg.max_length, vocab, cfg.seed, task=kind)
    val = synthetic_token_examples(n_val, cfg.max_length, vocab, cfg.seed + 1, task=kind)
    return batched(train), batched(val), tokenizer


def setup_sst2_data(config, vocab_size: int = 30522):
    """``(train_batches, val_batches, tokenizer)`` for the SST-2 protocol; random tokens when no corpus is cached."""
    return _loaders(config, vocab_size, "sst2")


def setup_wikitext_data(config, vocab_size: int = 50257):
    """``(train_batches, val_batches, tokenizer)`` of packed ``max_length`` blocks for the language-model protocol."""
    return _loaders(config, vocab_size, "wikitext103")


def create_bert_sst2(model_name: Optional[str] = None, **overrides) -> nn.Module:
    from stacr_b200.models import build_model

    return build_model(model_name or "bert-base-uncased", task="sequence_classification", **overrides)


def create_gpt2_lm(model_name: str = "gpt2", **overrides) -> nn.Module:
    """Any in-tree decoder preset (GPT-2, Pythia, Llama families) with a language-model head."""
    from stacr_b200.models import build_model

    return build_model(model_name, **overrides)


_MLP_ALL = ("mlp.c_fc", "mlp.c_proj", "mlp.dense_h_to_4h", "mlp.dense_4h_to_h", "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")
_MLP_WIDE_INPUT = ("mlp.c_proj", "mlp.dense_4h_to_h", "mlp.down_proj")


def get_compression_targets_gpt2(model: nn.Module, target_mode: str = "all") -> List[str]:
    """MLP projections of a decoder LM; ``largest_mlp_only`` keeps the ones whose input is the expanded width."""
    try:
        parts = {"all": _MLP_ALL, "largest_mlp_only": _MLP_WIDE_INPUT}[target_mode]
    except KeyError:
        raise ValueError(f"Unsupported decoder target mode: {target_mode}. Use 'all' or 'largest_mlp_only'.") from None
    return [name for name, _ in model.named_modules() if name.endswith(parts)]


def get_compression_targets_bert(model: nn.Module) -> List[str]:
    """Feed-forward output projections of a BERT encoder (``...output.dense`` outside the attention block)."""
    return [name for name, _ in model.named_modules() if name.endswith("output.dense") and "attention" not in name]


_RESHAPES = {512: (8, 8, 8), 768: (8, 8, 12), 1024: (8, 8, 16), 2048: (8, 16, 16), 3072: (12, 16, 16), 4096: (16, 16, 16)}


def auto_reshape_shape(in_features: int) -> Optional[Tuple[int, ...]]:
    """Three balanced factors of ``in_features`` (largest at most 4x the smallest) for the tensorised comparators."""
    if in_features in _RESHAPES:
        return _RESHAPES[in_features]
    for a in range(int(round(in_features ** (1.0 / 3.0))), 0, -1):
        if in_features % a:
            continue
        rest = in_features // a
        for b in range(int(round(math.sqrt(rest))), 0, -1):
            if rest % b:
                continue
            dims = sorted((a, b, rest // b))
            if dims[2] <= 4 * dims[0]:
                return tuple(reversed(dims))
    return None


def apply_min_adaptation_rule(stacr_cfg, max_steps: Optional[int], log_fn=print):
    """Switch a random-QR initialised basis to SVD init when the run freezes it before it could adapt.

    Applies when the basis starts random, is frozen after warm-up, gets fewer than ``min_adaptation_steps``
    updates, and ``allow_unadapted_random_qr`` is off.
    """
    if max_steps is None:
        return stacr_cfg
    steps = int(max_steps)
    if getattr(stacr_cfg, "freeze_basis_after_warmup", False):
        steps = min(steps, max(int(getattr(stacr_cfg, "warmup_steps", 0)), 0))
    if (getattr(stacr_cfg, "use_random_qr_init", False) and getattr(stacr_cfg, "freeze_basis_after_warmup", False)
            and steps < int(getattr(stacr_cfg, "min_adaptation_steps", 0)) and not getattr(stacr_cfg, "allow_unadapted_random_qr", False)):
        msg = (f"[min-adaptation] a random-QR basis would see only {steps} update step(s) before it is frozen "
               f"(< {stacr_cfg.min_adaptation_steps}); using SVD initialisation instead")
        warnings.warn(msg)
        if log_fn is not None:
            log_fn(msg)
        stacr_cfg.use_random_qr_init = False
    return stacr_cfg


# ------------------------------------------------------------------------------ storage estimators
def _batch_tokens(config, override: Optional[int] = None) -> int:
    if override is not None:
        return int(override)
    if getattr(config, "task", "") in ("sst2", "wikitext103"):
        return int(config.batch_size) * int(config.max_length)
    return int(config.batch_size)


def _summary(tokens, details) -> Optional[Dict[str, Any]]:
    if not details:
        return None
    stored = sum(int(d["stored_bytes"] or 0) for d in details)
    orig = sum(int(d["original_bytes"]) for d in details)
    return {"batch_tokens_est": tokens, "layers": len(details), "stored_bytes": stored or None, "original_bytes": orig or None,
            "achieved_ratio": (orig / stored) if stored else None, "layer_details": details}


def _activation_dtype(config) -> torch.dtype:
    name = str(getattr(getattr(config, "baseline_cfg", None), "amp_dtype", None) or getattr(config, "amp_dtype", "") or "")
    return {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16}.get(name, torch.float32)


def estimate_storage_for_model(model: nn.Module, config) -> Optional[Dict[str, Any]]:
    """Stored and dense bytes of every per-batch-factorised (``svd``/``tt``/``tucker``) layer for one batch."""
    from stacr_b200.protocols.layers import CompressedLinear

    if getattr(config, "method", "") == "baseline":
        return None
    tokens, dtype, details = _batch_tokens(config), _activation_dtype(config), []
    for name, layer in model.named_modules():
        if not isinstance(layer, CompressedLinear):
            continue
        lc = getattr(layer, "config", None) or {}
        method = lc.get("method", config.method)
        feats = layer.linear.in_features
        rank = int(lc.get("rank", config.rank) or 1)
        bits = lc.get("factor_quantization_bits", getattr(config, "factor_quantization_bits", None))
        dims = tuple(lc.get("reshape_shape") or ()) or auto_reshape_shape(feats) or (feats,)
        orig = tokens * feats * acct.bytes_per_elem(dtype)
        if method == "svd":
            stored = acct.svd_stored_bytes(tokens, feats, min(rank, tokens, feats), dtype).total_bytes
        elif method == "tt":
            full = (tokens,) + tuple(dims)
            stored = acct.tt_stored_bytes(full, lc.get("ranks") or acct.tt_uniform_ranks(full, rank), dtype).total_bytes
        elif method == "tucker":
            full = (tokens,) + tuple(dims)
            stored = acct.tucker_stored_bytes(full, lc.get("ranks") or acct.tucker_uniform_ranks(full, rank), dtype).total_bytes
        else:
            stored = None
        if stored is not None and bits:
            stored = int(math.ceil(stored * float(bits) / (8.0 * acct.bytes_per_elem(dtype))))
        details.append({"name": name, "method": method, "in_features": feats, "rank": rank, "stored_bytes": stored, "original_bytes": orig})
    return _summary(tokens, details)


def estimate_storage_for_stacr(model: nn.Module, config, actual_batch_tokens: Optional[int] = None) -> Optional[Dict[str, Any]]:
    """Stored and dense bytes of every STAC-R layer at its *active* rank and effective residual budget.

    ``actual_batch_tokens`` overrides the token count (full-batch graph training stores one row per node).  A layer
    on the low-rank-only route, or one whose residual budget is zero, is charged no residual.
    """
    import stacr_b200 as S
    from stacr_b200.adaptive import STACRLinear as AdaptiveLinear

    tokens, dtype, details = _batch_tokens(config, actual_batch_tokens), _activation_dtype(config), []
    for name, layer in model.named_modules():
        if not isinstance(layer, (AdaptiveLinear, S.STACRLinear)):
            continue
        lc = layer.config if hasattr(layer, "config") else None
        rank = int(layer.get_active_rank() if hasattr(layer, "get_active_rank") else getattr(layer, "rank", getattr(lc, "rank", 1)))
        budget = float(getattr(lc, "residual_budget", getattr(layer, "residual_budget", 0.0)) or 0.0)
        mode = getattr(lc, "residual_mode", "topk")
        state = getattr(layer, "layer_state", {}) or {}
        if mode == "none" or state.get("b1_route_active"):
            budget = 0.0
        cbits = getattr(lc, "quantize_bits", None) if getattr(lc, "quantize_coefficients", False) else None
        rbits = getattr(lc, "residual_quantize_bits", None) if getattr(lc, "quantize_residuals", False) else None
        if lc is None:                                    # projection engine: bf16 coefficients, int8 residual values
            rbits = getattr(layer, "residual_bits", 8)
        stored = acct.stacr_stored_bytes(tokens, layer.in_features, rank, budget, dtype, cbits, rbits)
        stored = int(stored.total_bytes)
        details.append({"name": name, "in_features": layer.in_features, "allocated_rank": int(getattr(lc, "rank", rank)), "active_rank": rank,
                        "residual_budget": budget, "stored_bytes": stored, "original_bytes": tokens * layer.in_features * acct.bytes_per_elem(dtype)})
    return _summary(tokens, details)


def estimate_storage_for_c1(model: nn.Module, config, actual_batch_tokens: Optional[int] = None) -> Optional[Dict[str, Any]]:
    """Stored and dense bytes of the checkpoint-boundary compressor: quantised coefficients per registered site."""
    from stacr_b200.protocols.checkpointing import get_active_c1_runtime, get_global_checkpoint_site_registry

    runtime = get_active_c1_runtime()
    registry = runtime.registry if runtime is not None else get_global_checkpoint_site_registry()
    specs = list(registry.specs())
    if not specs:
        return None
    tokens, dtype, details = _batch_tokens(config, actual_batch_tokens), _activation_dtype(config), []
    for spec in specs:
        bits = spec.quantize_bits if spec.quantize_coefficients else None
        stored = acct.stacr_ckpt_stored_bytes(tokens, spec.hidden_size, spec.rank, dtype, coeff_bits=bits)
        details.append({"name": spec.site_id, "in_features": spec.hidden_size, "rank": spec.rank, "stored_bytes": int(stored),
                        "original_bytes": tokens * spec.hidden_size * acct.bytes_per_elem(dtype)})
    return _summary(tokens, details)


def estimate_storage_for_prac(model: nn.Module, config, actual_batch_tokens: Optional[int] = None) -> Optional[Dict[str, Any]]:
    """Stored and dense bytes of every PRAC layer: ``tokens x rank`` coefficients; the projection is a persistent buffer."""
    from stacr_b200.protocols.prac import PRACLinear

    tokens, dtype, details = _batch_tokens(config, actual_batch_tokens), _activation_dtype(config), []
    for name, layer in model.named_modules():
        if isinstance(layer, PRACLinear):
            per = acct.bytes_per_elem(dtype)
            details.append({"name": name, "in_features": layer.in_features, "rank": layer.effective_rank,
                            "stored_bytes": tokens * layer.effective_rank * per, "original_bytes": tokens * layer.in_features * per,
                            "projection_buffer_bytes": int(layer.projection_buffer_bytes())})
    out = _summary(tokens, details)
    if out:
        out["persistent_projection_bytes"] = sum(d["projection_buffer_bytes"] for d in details)
    return out


# ------------------------------------------------------------------------------ baselines and the epoch loop
@dataclass
class BaselineState:
    """What ``apply_baseline`` switched on, in attribute form (the runner itself uses the equivalent mapping)."""

    amp_manager: Optional[Any] = None
    offloader: Optional[Any] = None
    gact_controller: Optional[Any] = None
    c1_runtime: Optional[Any] = None
    status: str = "enabled"
    reason: Optional[str] = None

    @classmethod
    def from_mapping(cls, state: Dict[str, Any]) -> "BaselineState":
        return cls(amp_manager=state.get("amp"), offloader=state.get("offload"), gact_controller=state.get("gact"),
                   c1_runtime=state.get("c1_runtime"), status=state.get("status", "enabled"), reason=state.get("reason"))


def train_epoch(model: nn.Module, train_loader, criterion, optimizer, scheduler, device, config, epoch: int, logger,
                amp_manager=None, gact_controller=None, offloader=None, compressor=None, accum_steps: int = 1,
                grad_clip: float = 0.0, global_step_offset: int = 0) -> Dict[str, float]:
    """One pass over ``train_loader`` (an iterable of ``input_ids``/``labels`` mappings), stopping at ``config.max_steps``.

    The model's own loss is used when it returns one; otherwise ``criterion(logits, labels)``.  Returns the mean
    loss, accuracy (classification), tokens/s and ``steps_completed`` (optimizer steps of this epoch).
    """
    import contextlib

    import stacr_b200 as S
    from stacr_b200.adaptive import set_stacr_runtime_state

    model.train()
    accum = max(1, int(accum_steps))
    limit = getattr(config, "max_steps", None)
    layers = [m for m in model.modules() if isinstance(m, S.STACRLinear)]
    optimizer.zero_grad(set_to_none=True)
    started = time.perf_counter()
    loss_sum, seen, correct, tokens, steps, micro = 0.0, 0, 0, 0, 0, 0
    for batch in train_loader:
        step = global_step_offset + steps
        if limit is not None and step >= int(limit):
            break
        batch = {k: v.to(device) for k, v in batch.items() if isinstance(v, torch.Tensor)}
        S.set_step(layers, step)
        set_stacr_runtime_state(model, step, micro % accum, accum, limit)
        cast = amp_manager.autocast() if amp_manager is not None else contextlib.nullcontext()
        hold = offloader.training_step() if offloader is not None and hasattr(offloader, "training_step") else contextlib.nullcontext()
        with hold:
            with cast:
                out = model(**batch)
                loss = out.loss if getattr(out, "loss", None) is not None else criterion(out.logits, batch["labels"])
            (amp_manager.backward if amp_manager is not None else torch.Tensor.backward)(loss / accum)
        value = float(loss.detach())
        if not math.isfinite(value):
            raise FloatingPointError(f"Nonfinite loss at epoch {epoch}, step {step}")
        n = batch["input_ids"].shape[0]
        loss_sum += value * n
        seen += n
        tokens += int(batch["attention_mask"].sum()) if "attention_mask" in batch else batch["input_ids"].numel()
        if batch["labels"].dim() == 1 and getattr(out, "logits", None) is not None:
            correct += int((out.logits.argmax(-1) == batch["labels"]).sum())
        micro += 1
        if micro % accum == 0:
            if grad_clip and grad_clip > 0:
                if amp_manager is not None:
                    amp_manager.unscale_(optimizer)
                torch.nn.utils.clip_grad_norm_(model.parameters(), grad_clip)
            amp_manager.step(optimizer) if amp_manager is not None else optimizer.step()
            if scheduler is not None:
                scheduler.step()
            optimizer.zero_grad(set_to_none=True)
            if logger is not None and hasattr(logger, "log"):
                logger.log({"epoch": epoch, "step": step, "train_loss": value})
            steps += 1
    wall = time.perf_counter() - started
    return {"train_loss": loss_sum / max(seen, 1), "train_acc": correct / max(seen, 1), "tokens_per_sec": tokens / wall if wall > 0 else 0.0,
            "epoch_time_s": wall, "steps_completed": steps, "total_tokens": tokens}
