"""Generic trainer and same-batch gradient-fidelity protocol.

Config vocabulary, method names, composition rules and result fields follow
stacr/training.py:21-668 of the reference project, so its YAML presets run unchanged.  Differences:
``dataset: synthetic`` / ``random_init: true`` build in-tree random-init models and uniform-random
token batches (no network); ``optimizer: adamw8bit`` uses the in-tree block-wise 8-bit AdamW
instead of an external library; timing uses CUDA events; ``resume_from`` restores a checkpoint
written through ``checkpoint_path`` (model, optimizer, step, RNG).
"""

from __future__ import annotations

import copy
import importlib
import math
import time
from pathlib import Path
from typing import Any, NamedTuple

import torch

from .surgery import _SELECTION_KEYS, apply_stacr, select_target_names, set_step
from .utils import device_from_config, set_seed, write_csv

class _Method(NamedTuple):
    """What a method name stands for; the trainer reads these flags, never the name's spelling."""

    compresses: bool = False              # wraps linear layers with STAC-R
    turbo: bool = False                   # residual channel switched off after ``turbo_after_step`` (default 50)
    optimizer_family: str | None = None   # low-rank-gradient optimizer the method is defined with
    checkpoints: bool = False             # activation checkpointing on a block stride


_METHOD_TABLE = {
    "baseline": _Method(),
    "freeze": _Method(),
    "checkpointing": _Method(checkpoints=True),
    "galore": _Method(optimizer_family="galore"),
    "subtrack": _Method(optimizer_family="subtrack"),
    "stacr": _Method(compresses=True),
    "turbofast": _Method(compresses=True, turbo=True),
    "stacr_galore": _Method(compresses=True, optimizer_family="galore"),
    "turbofast_galore": _Method(compresses=True, turbo=True, optimizer_family="galore"),
    "subtrack_stacr": _Method(compresses=True, optimizer_family="subtrack"),
    "stacr_checkpointing": _Method(compresses=True, checkpoints=True),
    "turbofast_checkpointing": _Method(compresses=True, turbo=True, checkpoints=True),
}
STACR_METHODS = {name for name, spec in _METHOD_TABLE.items() if spec.compresses}
METHODS = set(_METHOD_TABLE)
_FAMILY_LABEL = {"galore": "GaLore", "subtrack": "SubTrack"}
TASKS = ("synthetic", "language_modeling", "sequence_classification")

# keys handed to the wrapped layers / the layer selection
CORE_KEYS = (
    "rank", "residual_budget", "residual_bits", "oja_lr", "update_interval", "warmup_steps", "freeze_after_warmup",
    "turbo_after_step", "chunk_rows", "basis_dtype", "residual_mode", "residual_block_size", "residual_sample_ratio", "surface",
    "min_features", "extra_names", "target_names", "target_pattern", "exclude_names", "trainable_only", "allow_empty",
)
# keys of the run itself, grouped by what reads them
RUN_KEYS = {
    # what is trained, on what
    "task", "method", "engine", "compression", "model_name", "model_revision", "model_dtype", "attn_implementation", "local_files_only",
    "dataset", "dataset_revision", "train_file", "validation_file", "max_examples", "max_eval_examples", "features", "hidden",
    # the loop
    "device", "seed", "steps", "batch_size", "seq_len", "gradient_accumulation_steps", "measure_from", "fidelity_steps", "amp",
    # optimisation
    "lr", "weight_decay", "optimizer", "use_8bit_optimizer", "lr_warmup_steps", "lr_schedule", "max_grad_norm",
    "galore_rank", "galore_update_proj_gap", "galore_scale", "galore_proj_type", "galore_target_modules",
    "subtrack_rank", "subtrack_scale", "subtrack_update_interval", "subtrack_step_size", "subtrack_target_modules",
    "subtrack_proj_type", "subtrack_adaptive_optimizer", "subtrack_recovery_scaling", "subtrack_norm_growth_limit",
    # composition with checkpointing / offload, and the saved state
    "checkpoint_path", "checkpoint_every", "checkpoint_offset", "offload_every", "offload_offset", "compression_blocks",
    "attention_surface", "freeze_basis_after_warmup",
    # additions of this framework
    "random_init", "vocab_size", "resume_from", "model_overrides",
}
_PER_TASK_DEFAULTS = {
    True: {"method": "turbofast", "steps": 5, "batch_size": 8},       # synthetic
    False: {"method": "baseline", "steps": 500, "batch_size": 2},     # Hugging Face tasks
}
_SHARED_DEFAULTS = {"seed": 42, "gradient_accumulation_steps": 1, "measure_from": 0, "engine": "projection"}


def _range_problems(cfg: dict):
    """Yield ``(violated, message)`` in the order the checks are reported."""
    yield cfg["engine"] not in ("projection", "adaptive"), "engine must be projection or adaptive"
    yield cfg["method"] not in METHODS, f"Unknown method {cfg['method']!r}; choose from {sorted(METHODS)}"
    yield cfg["task"] not in TASKS, f"Unknown task {cfg['task']!r}"
    for key in ("steps", "batch_size", "gradient_accumulation_steps"):
        yield int(cfg[key]) < 1, f"{key} must be positive"
    yield not 0 <= int(cfg["measure_from"]) < int(cfg["steps"]), "measure_from must be in [0, steps)"
    yield cfg["task"] != "synthetic" and not cfg.get("model_name"), "model_name is required for Hugging Face training"


def validate_config(config: dict) -> dict:
    """A copy of ``config`` with task- and method-dependent defaults filled in; unknown keys, names and ranges are rejected."""
    cfg = copy.deepcopy(config)
    unknown = sorted(set(cfg) - RUN_KEYS - set(CORE_KEYS))
    if unknown:
        raise ValueError(f"Unknown training configuration fields: {unknown}")
    cfg.setdefault("task", "synthetic")
    for key, value in {**_PER_TASK_DEFAULTS[cfg["task"] == "synthetic"], **_SHARED_DEFAULTS}.items():
        cfg.setdefault(key, value)
    for violated, message in _range_problems(cfg):
        if violated:
            raise ValueError(message)
    spec = _METHOD_TABLE[cfg["method"]]
    if spec.compresses:
        cfg.setdefault("turbo_after_step", 50 if spec.turbo else None)
    if spec.optimizer_family:
        if cfg.setdefault("optimizer", spec.optimizer_family) != spec.optimizer_family:
            raise ValueError(f"A {_FAMILY_LABEL[spec.optimizer_family]} method requires optimizer={spec.optimizer_family}")
    if spec.checkpoints:
        cfg.setdefault("checkpoint_every", 2 if spec.compresses else 1)
    return cfg


# ---------------------------------------------------------------------------------------------- layer options
def _projection_options(cfg: dict) -> dict:
    """Layer options of the projection engine: the core keys present, then the ``compression`` mapping, then the two aliases."""
    opts = {key: cfg[key] for key in CORE_KEYS if key in cfg}
    if cfg.get("engine", "projection") == "projection":
        opts.update(cfg.get("compression", {}))
    if cfg.get("attention_surface"):
        opts["surface"] = "mlp+attention"
    if "freeze_basis_after_warmup" in cfg:
        opts["freeze_after_warmup"] = cfg["freeze_basis_after_warmup"]
    return opts


_ADAPTIVE_PASSTHROUGH = ("basis_dtype", "update_interval", "warmup_steps", "residual_block_size", "residual_mode")
_ADAPTIVE_RENAMED = {"oja_lr": "oja_learning_rate", "chunk_rows": "chunk_size", "freeze_after_warmup": "freeze_basis_after_warmup"}
_ADAPTIVE_TURBO = {"post_warmup_residual_mode": "none", "refresh_trigger": "residual_energy", "cache_basis_per_optimizer_step": True,
                   "oja_update_per_optimizer_step": True}


def _adaptive_options(cfg: dict, core: dict) -> dict:
    """The same settings in the adaptive engine's vocabulary (``compression`` entries, already in that vocabulary, win)."""
    opts = {key: value for key, value in core.items() if key in _SELECTION_KEYS}
    opts.update(rank=int(cfg.get("rank", 8)), residual_budget=float(cfg.get("residual_budget", 0.005)))
    opts.update({key: cfg[key] for key in _ADAPTIVE_PASSTHROUGH if key in cfg})
    opts.update({theirs: core[ours] for ours, theirs in _ADAPTIVE_RENAMED.items() if ours in core})
    bits = cfg.get("residual_bits")
    if bits is not None:
        if bits not in (0, 4, 8):
            raise ValueError("residual_bits must be 0, 4, or 8")
        opts["quantize_residuals"] = bits != 0
        if bits:
            opts["residual_quantize_bits"] = bits
    if "residual_sample_ratio" in cfg:
        raise ValueError("The adaptive engine uses compression.streaming_topk_sample_ratio for threshold sampling")
    if _METHOD_TABLE[cfg["method"]].turbo:
        opts.update(_ADAPTIVE_TURBO, residual_warmup_steps=int(cfg["turbo_after_step"]))
    opts.update(cfg.get("compression", {}))
    return opts


# ---------------------------------------------------------------------------------------------- composition
def _strided_blocks(n_blocks: int, every: int, offset: int, what: str) -> list[int]:
    """Block indices ``offset, offset + every, ...`` of a ``what`` plan (``every == 0``: none)."""
    if not every:
        return []
    if not 0 <= offset < every:
        raise ValueError(f"{what}_offset must be in [0, {what}_every)")
    return list(range(offset, n_blocks, every))


def _selection_of(options: dict) -> dict:
    return {key: value for key, value in options.items() if key in _SELECTION_KEYS and key != "allow_empty"}


def configure_model(model, config: dict):
    """Plan, then mutate: freeze -> wrap -> checkpoint -> offload, before any optimizer or gradient synchroniser is built.

    With ``compression_blocks: complement`` (the default) a STAC-R method wraps only the blocks that are *not* checkpointed:
    a checkpointed block recomputes its activations anyway, so compressing them would cost time and save nothing.
    """
    from .composition import block_target_names, checkpoint_blocks, offload_blocks, transformer_blocks

    cfg = validate_config(config)
    spec = _METHOD_TABLE[cfg["method"]]
    options = _projection_options(cfg)
    if cfg["task"] == "synthetic":
        options.setdefault("surface", "all")
        options.setdefault("min_features", 1)
    if cfg["engine"] == "adaptive":
        options = _adaptive_options(cfg, options)
    scope = cfg.get("compression_blocks", "complement")
    if scope not in ("complement", "all"):
        raise ValueError("compression_blocks must be 'complement' or 'all'")
    strides = {what: int(cfg.get(f"{what}_every", 0)) for what in ("checkpoint", "offload")}
    if min(strides.values()) < 0:
        raise ValueError("checkpoint_every and offload_every must be nonnegative")

    # ---- plan (nothing is modified yet)
    blocks = transformer_blocks(model) if any(strides.values()) else None
    n_blocks = len(blocks) if blocks is not None else 0
    checkpointed = _strided_blocks(n_blocks, strides["checkpoint"], int(cfg.get("checkpoint_offset", 0)), "checkpoint")
    if checkpointed and spec.compresses and scope == "complement":
        remaining = block_target_names(model, blocks, lambda index: index not in checkpointed, **_selection_of(options))
        if not remaining:
            raise ValueError("No uncheckpointed STAC-R surface remains; use selective checkpointing")
        options = {key: value for key, value in options.items() if key not in _SELECTION_KEYS}
        options.update(surface="none", target_names=remaining)
    offloaded = _strided_blocks(n_blocks, strides["offload"], int(cfg.get("offload_offset", 0)), "offload")
    frozen: list[str] = []
    if cfg["method"] == "freeze":
        frozen = select_target_names(model, **_selection_of(options))
        if not frozen:
            raise ValueError("No modules selected for the freeze control")

    # ---- apply
    for name in frozen:
        model.get_submodule(name).requires_grad_(False)
    layers: list = []
    if spec.compresses:
        if cfg["engine"] == "adaptive":
            from .adaptive import apply_adaptive_stacr as wrap
        else:
            wrap = apply_stacr
        layers = wrap(model, options)
    if checkpointed:
        checkpoint_blocks(blocks, checkpointed)
    if offloaded:
        offload_blocks(blocks, offloaded)
    return layers, {"checkpointed_blocks": checkpointed, "offloaded_blocks": offloaded, "wrapped_names": [layer.source_name for layer in layers]}


def _build_optimizer(model, config):
    lr = float(config.get("lr", 5e-5))
    decay = float(config.get("weight_decay", 0.0))
    name = str(config.get("optimizer", "adamw8bit" if config.get("use_8bit_optimizer") else "adamw")).lower()
    params = [p for p in model.parameters() if p.requires_grad]
    if not params:
        raise ValueError("The model has no trainable parameters")
    if name == "adamw":
        if params[0].is_cuda:
            from .optim import AdamW

            return AdamW(params, lr=lr, weight_decay=decay), "AdamW"
        return torch.optim.AdamW(params, lr=lr, weight_decay=decay), "AdamW"
    if name == "adamw8bit":
        from .optim import AdamW8bit

        return AdamW8bit(params, lr=lr, weight_decay=decay), "AdamW8bit"
    if name == "galore":
        from .comparators.galore_adapter import create_galore_optimizer

        return create_galore_optimizer(
            model, lr=lr, rank=int(config.get("galore_rank", 128)), update_proj_gap=int(config.get("galore_update_proj_gap", 200)),
            scale=float(config.get("galore_scale", 0.25)), proj_type=config.get("galore_proj_type", "std"), weight_decay=decay,
            target_modules=config.get("galore_target_modules"),
        ), "GaLoreAdamW"
    if name == "subtrack":
        from .comparators.subtrack_adapter import create_subtrack_optimizer

        return create_subtrack_optimizer(model, config), "SubTrack++"
    if ":" in name:
        module, attr = str(config["optimizer"]).split(":", 1)
        opt = getattr(importlib.import_module(module), attr)(model, config)
        if not isinstance(opt, torch.optim.Optimizer):
            raise TypeError("Optimizer factory must return torch.optim.Optimizer")
        return opt, str(config["optimizer"])
    raise ValueError(f"Unknown optimizer {name!r}")


def _amp_dtype(config, device):
    mode = str(config.get("amp", "none")).lower()
    if mode in ("none", "off", "false"):
        return None
    if mode in ("bf16", "bfloat16"):
        if device.type == "cuda" and not torch.cuda.is_bf16_supported():
            raise ValueError("bf16 was requested but this CUDA device does not support it")
        return torch.bfloat16
    if mode in ("fp16", "float16"):
        if device.type != "cuda":
            raise ValueError("fp16 training requires CUDA; use bf16 or none on CPU")
        return torch.float16
    raise ValueError("amp must be none, bf16 or fp16")


def _sync(device):
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def _lr_fraction(step: int, steps: int, warmup: int, schedule: str) -> float:
    if step < warmup or schedule == "constant":
        return min(1.0, (step + 1) / max(1, warmup))
    progress = (step - warmup) / max(1, steps - warmup - 1)
    return 1 - progress if schedule == "linear" else (1 + math.cos(math.pi * progress)) / 2


@torch.no_grad()
def _evaluate(model, loader, device, task, amp_dtype):
    was_training = model.training
    model.eval()
    nll_sum = tokens = hits = seen = tp = fp = fn = 0
    try:
        for batch in loader:
            batch = {k: v.to(device) for k, v in batch.items()}
            with torch.autocast(device_type=device.type, dtype=amp_dtype, enabled=amp_dtype is not None):
                out = model(**batch)
            if task == "sequence_classification":
                pred, gold = out.logits.argmax(-1), batch["labels"]
                hits += int((pred == gold).sum())
                seen += gold.numel()
                tp += int(((pred == 1) & (gold == 1)).sum())
                fp += int(((pred == 1) & (gold != 1)).sum())
                fn += int(((pred != 1) & (gold == 1)).sum())
            else:
                n = int((batch["labels"][..., 1:] != -100).sum())
                nll_sum += float(out.loss) * n
                tokens += n
    finally:
        model.train(was_training)
    if task == "sequence_classification":
        if not seen:
            raise ValueError("Validation dataset is empty")
        return {"accuracy": 100 * hits / seen, "f1": 100 * 2 * tp / max(1, 2 * tp + fp + fn), "ppl": None}
    if not tokens:
        raise ValueError("Validation dataset has no nonmasked causal targets")
    nll = nll_sum / tokens
    return {"accuracy": None, "ppl": math.exp(nll) if nll < 709 else float("inf"), "nll": nll}


def train_model(model, train_batches, config: dict, *, validation_batches=None) -> dict:
    """Train any model that returns ``.loss`` on dict batches.  ``steps`` counts optimizer updates."""
    cfg = validate_config(config)
    device = device_from_config(cfg.get("device", "auto"))
    if not len(train_batches):
        raise ValueError("Training dataset is empty")
    model.to(device).train()
    layers, composition = configure_model(model, cfg)
    optimizer, optimizer_name = _build_optimizer(model, cfg)
    dtype = _amp_dtype(cfg, device)
    scaler = torch.amp.GradScaler(device.type, enabled=dtype is torch.float16)
    steps, accum = int(cfg["steps"]), int(cfg["gradient_accumulation_steps"])
    measure_from, warmup = int(cfg["measure_from"]), int(cfg.get("lr_warmup_steps", 0))
    schedule = cfg.get("lr_schedule", "constant")
    if not 0 <= warmup <= steps:
        raise ValueError("lr_warmup_steps must be between zero and steps")
    if schedule not in ("constant", "linear", "cosine"):
        raise ValueError("lr_schedule must be constant, linear or cosine")
    first_step = 0
    if cfg.get("resume_from"):
        from .parallel.health import load_checkpoint

        blob = load_checkpoint(cfg["resume_from"], map_location=device)  # refuses a truncated or altered file
        model.load_state_dict(blob["model"])
        optimizer.load_state_dict(blob["optimizer"])
        scaler.load_state_dict(blob.get("scaler", {}))
        first_step = int(blob.get("step", 0))
        if "rng_state" in blob:
            torch.set_rng_state(blob["rng_state"].cpu())
    base_lr = [g["lr"] for g in optimizer.param_groups]
    losses: list[float] = []
    tokens = measured = 0
    wall0 = None
    ev0 = ev1 = None
    for step in range(first_step, steps):
        if step == max(measure_from, first_step):
            _sync(device)
            if device.type == "cuda":
                torch.cuda.reset_peak_memory_stats(device)
                ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ev0.record()
            wall0 = time.perf_counter()
        frac = _lr_fraction(step, steps, warmup, schedule)
        for group, lr in zip(optimizer.param_groups, base_lr):
            group["lr"] = lr * frac
        optimizer.zero_grad(set_to_none=True)
        loss_acc = 0.0
        for micro in range(accum):
            set_step(layers, step, microbatch_index=micro, accum_steps=accum)
            batch = train_batches[(step * accum + micro) % len(train_batches)]
            batch = {k: v.to(device, non_blocking=True) for k, v in batch.items()}
            with torch.autocast(device_type=device.type, dtype=dtype, enabled=dtype is not None):
                loss = model(**batch).loss
            if not torch.isfinite(loss).all():
                raise FloatingPointError(f"Nonfinite loss at optimizer step {step}")
            scaler.scale(loss / accum).backward()
            loss_acc += float(loss.detach()) / accum
            if step >= measure_from and "input_ids" in batch:
                tokens += int(batch.get("attention_mask", torch.ones_like(batch["input_ids"])).sum())
        if cfg.get("max_grad_norm") is not None:
            scaler.unscale_(optimizer)
            torch.nn.utils.clip_grad_norm_(model.parameters(), float(cfg["max_grad_norm"]))
        scaler.step(optimizer)
        scaler.update()
        if device.type == "cuda":
            from .ops import _lib

            _lib.poll_status(device)      # a kernel that gave up on a bounded wait during this or the previous step raises here
        losses.append(loss_acc)
        if step >= measure_from:
            measured += 1
    peak = reserved = None
    if device.type == "cuda" and ev0 is not None:
        ev1.record()
        _sync(device)
        elapsed = ev0.elapsed_time(ev1) / 1e3
        peak = torch.cuda.max_memory_allocated(device) / 1024**3
        reserved = torch.cuda.max_memory_reserved(device) / 1024**3
    else:
        _sync(device)
        elapsed = time.perf_counter() - (wall0 if wall0 is not None else time.perf_counter())
    result = {
        "task": cfg["task"], "model": cfg.get("model_name", "synthetic"), "method": cfg["method"], "engine": cfg["engine"],
        "optimizer": optimizer_name, "steps": steps, "steps_measured": measured, "batch_size": int(cfg["batch_size"]),
        "gradient_accumulation_steps": accum, "seq_len": cfg.get("seq_len"), "seed": int(cfg["seed"]),
        "wrapped_layers": len(layers), "train_loss": losses[-1] if losses else None, "first_loss": losses[0] if losses else None,
        "peak_gib": peak, "reserved_gib": reserved, "seconds": elapsed,
        "tokens_per_second": tokens / elapsed if tokens and elapsed > 0 else None, "amp": cfg.get("amp", "none"),
        "device": str(device), "torch_version": torch.__version__, **composition,
    }
    if validation_batches is not None:
        quality = _evaluate(model, validation_batches, device, cfg["task"], dtype)
        result.update({f"val_{k}": v for k, v in quality.items()})
    if cfg.get("checkpoint_path"):
        target = Path(cfg["checkpoint_path"])
        target.parent.mkdir(parents=True, exist_ok=True)
        from .parallel.health import write_checkpoint

        write_checkpoint(
            {
                "model": model.state_dict(), "optimizer": optimizer.state_dict(), "scaler": scaler.state_dict(), "step": steps,
                "config": cfg, "rng_state": torch.get_rng_state(),
                "cuda_rng_state": torch.cuda.get_rng_state_all() if device.type == "cuda" else [],
            },
            target,
        )
    return result


def run_synthetic(config):
    """Two-layer GELU autoencoder on Gaussian batches (the reference's synthetic task)."""
    from types import SimpleNamespace

    cfg = validate_config(config)
    set_seed(cfg["seed"])
    features, hidden = int(cfg.get("features", 64)), int(cfg.get("hidden", 32))

    class Autoencoder(torch.nn.Sequential):
        def forward(self, inputs, labels):
            out = super().forward(inputs)
            return SimpleNamespace(loss=(out - labels).square().mean(), logits=out)

    model = Autoencoder(torch.nn.Linear(features, hidden), torch.nn.GELU(), torch.nn.Linear(hidden, features))
    gen = torch.Generator().manual_seed(int(cfg["seed"]) + 1)
    batches = []
    for _ in range(int(cfg["steps"]) * int(cfg["gradient_accumulation_steps"])):
        x = torch.randn(int(cfg["batch_size"]), features, generator=gen)
        batches.append({"inputs": x, "labels": x.clone()})
    return train_model(model, batches, cfg)


def _collate(examples: list[dict], batch_size: int) -> list[dict]:
    out = []
    for lo in range(0, len(examples) - batch_size + 1, batch_size):
        group = examples[lo:lo + batch_size]
        out.append({k: torch.stack([torch.as_tensor(ex[k]) for ex in group]) for k in group[0]})
    return out


def _hf_inputs(config):
    from .datasets import build_examples
    from .models import load_model_and_tokenizer

    dtype_name = str(config.get("model_dtype", "float32"))
    if dtype_name not in ("float32", "float16", "bfloat16"):
        raise ValueError("model_dtype must be float32, float16 or bfloat16")
    synthetic = config.get("dataset", "synthetic") == "synthetic"
    model, tokenizer = load_model_and_tokenizer(
        config["model_name"], config["task"], revision=config.get("model_revision"),
        attn_implementation=config.get("attn_implementation"), dtype=getattr(torch, dtype_name),
        local_files_only=bool(config.get("local_files_only", False)), random_init=bool(config.get("random_init", synthetic)),
    )
    if "vocab_size" not in config and hasattr(getattr(model, "config", None), "vocab_size"):
        config = {**config, "vocab_size": model.config.vocab_size}
    bs = int(config["batch_size"])
    train = _collate(build_examples(config, tokenizer), bs)
    validation = _collate(build_examples(config, tokenizer, validation=True), bs)
    return model, train, validation


def run_hf(config):
    cfg = validate_config(config)
    set_seed(cfg["seed"])
    model, train, validation = _hf_inputs(cfg)
    return train_model(model, train, cfg, validation_batches=validation or None)


def gradient_fidelity(config):
    """Cosine between uncompressed and compressed gradients on the same batch and weights.

    Before each measurement one dropout-free forward fits or refreshes the bases; the two measured
    passes run under ``compression_diagnostics`` and change neither compression state nor weights.
    """
    from .diagnostics import compression_diagnostics

    cfg = validate_config(config)
    set_seed(cfg["seed"])
    reference, batches, _ = _hf_inputs(cfg)
    test = copy.deepcopy(reference)
    device = device_from_config(cfg.get("device", "auto"))
    reference.to(device).train()
    test.to(device).train()
    paired = dict(test.named_parameters())  # wrappers keep Parameter identity, names may gain nesting
    layers, _ = configure_model(test, {**cfg, "method": "stacr"})
    dtype = _amp_dtype(cfg, device)
    steps = int(cfg.get("fidelity_steps", cfg["steps"]))
    if steps < 1:
        raise ValueError("fidelity_steps must be positive")
    wrapped = {layer.source_name + ".weight" for layer in layers}
    whole, local = [], []
    worst_other = 1.0

    def cosine(dot, na, nb):
        return dot / math.sqrt(na * nb) if na * nb > 0 else (1.0 if na == nb else 0.0)

    for step in range(steps):
        batch = {k: v.to(device) for k, v in batches[step % len(batches)].items()}
        set_step(layers, step)
        flags = {m: m.training for m in test.modules()}
        try:
            test.eval()
            for layer in layers:
                layer.training = True
            with torch.autocast(device_type=device.type, dtype=dtype, enabled=dtype is not None):
                test(**batch)
        finally:
            for m, flag in flags.items():
                m.training = flag
        for model in (reference, test):
            model.zero_grad(set_to_none=True)
            set_seed(int(cfg["seed"]) * 100003 + step + 1)
            with compression_diagnostics(model):
                with torch.autocast(device_type=device.type, dtype=dtype, enabled=dtype is not None):
                    loss = model(**batch).loss
                loss.backward()
        dot = n_ref = n_test = 0.0
        for name, p in reference.named_parameters():
            ga, gb = p.grad, paired[name].grad
            if ga is None or gb is None:
                if (ga is None) != (gb is None):
                    raise RuntimeError(f"Gradient presence differs at {name}")
                continue
            a, b = ga.double(), gb.double()
            d, na, nb = float((a * b).sum()), float(a.square().sum()), float(b.square().sum())
            dot, n_ref, n_test = dot + d, n_ref + na, n_test + nb
            if name in wrapped:
                local.append(cosine(d, na, nb))
            else:
                worst_other = min(worst_other, cosine(d, na, nb))
        whole.append(cosine(dot, n_ref, n_test))
    return {
        "model": cfg["model_name"], "steps": steps, "wrapped_layers": len(layers), "mean_cosine": sum(whole) / len(whole),
        "worst_cosine": min(whole), "local_mean_cosine": sum(local) / len(local) if local else None,
        "local_worst_cosine": min(local) if local else None, "worst_unwrapped_cosine": worst_other,
        "protocol": "eval_same_batch_frozen_compression_state", "basis_fit": "preceding_dropout_disabled_forward",
    }


def run_config(config: dict[str, Any]) -> dict[str, Any]:
    cfg = validate_config(config)
    return run_synthetic(cfg) if cfg["task"] == "synthetic" else run_hf(cfg)


def run_many(configs, output_csv):
    rows = [run_config(cfg) for cfg in configs]
    write_csv(output_csv, rows)
    return rows
