"""Sequence-classification fine-tuning with a low-rank-state optimizer (SubTrack, GaLore or plain AdamW), with or
without STAC-R on the encoder's feed-forward output projections.

This is the optimizer-state x activation composition protocol: the optimizer compresses *its* state, STAC-R the
saved activations, and the run reports accuracy, loss, throughput and peak memory for each combination.

    python -m stacr_b200.comparators.subtrack_protocol --enable_low_rank --low_rank_method subtrack --lora_r 8 \
        --enable_stacr --stacr_rank 8 --max_train_steps 50 --output_dir runs/subtrack_stacr

Parity: comparators/subtrack_protocol.py (flags ``--task_name --max_length --model_name_or_path
--per_device_train_batch_size --learning_rate --weight_decay --num_train_epochs --max_train_steps
--gradient_accumulation_steps --lr_scheduler_type --num_warmup_steps --output_dir --seed --enable_low_rank --lora_r
--subspace_update_interval --low_rank_scale --proj_type --low_rank_method --st_init_step_size --enable_stacr
--stacr_rank --stacr_residual_budget --stacr_residual_mode``; writes ``all_results.json``).  The reference drives
``accelerate`` and downloads GLUE; this version uses the in-tree BERT and optimizers and falls back to a synthetic
task of the same shapes when GLUE is not cached.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import time
from types import SimpleNamespace

import torch

GLUE_LABELS = {"cola": 2, "sst2": 2, "mrpc": 2, "qqp": 2, "mnli": 3, "qnli": 2, "rte": 2, "wnli": 2, "stsb": 1}


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="Low-rank optimizer x STAC-R composition on a GLUE-shaped task")
    p.add_argument("--task_name", default="sst2", choices=sorted(GLUE_LABELS))
    p.add_argument("--max_length", type=int, default=128)
    p.add_argument("--model_name_or_path", default="bert-base-uncased")
    p.add_argument("--model_overrides", default=None, help="JSON of architecture overrides (smaller depth/width for smoke runs)")
    p.add_argument("--per_device_train_batch_size", type=int, default=16)
    p.add_argument("--per_device_eval_batch_size", type=int, default=32)
    p.add_argument("--learning_rate", type=float, default=2e-5)
    p.add_argument("--weight_decay", type=float, default=0.0)
    p.add_argument("--num_train_epochs", type=int, default=3)
    p.add_argument("--max_train_steps", type=int, default=None)
    p.add_argument("--gradient_accumulation_steps", type=int, default=1)
    p.add_argument("--lr_scheduler_type", default="linear", choices=["linear", "cosine", "constant"])
    p.add_argument("--num_warmup_steps", type=int, default=0)
    p.add_argument("--train_examples", type=int, default=512)
    p.add_argument("--eval_examples", type=int, default=128)
    p.add_argument("--output_dir", default=None)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--device", default=None)
    p.add_argument("--enable_low_rank", action="store_true")
    p.add_argument("--low_rank_method", default="subtrack", choices=["subtrack", "galore"])
    p.add_argument("--lora_r", type=int, default=8, help="rank of the optimizer-state subspace")
    p.add_argument("--subspace_update_interval", type=int, default=200)
    p.add_argument("--low_rank_scale", type=float, default=0.25)
    p.add_argument("--proj_type", default="std")
    p.add_argument("--st_init_step_size", type=float, default=0.1, help="Grassmannian step size of the subspace tracker")
    p.add_argument("--enable_stacr", action="store_true")
    p.add_argument("--stacr_rank", type=int, default=8)
    p.add_argument("--stacr_residual_budget", type=float, default=0.005)
    p.add_argument("--stacr_residual_mode", default="topk", choices=["topk", "none", "block", "threshold"])
    p.add_argument("--disable_wandb", action="store_true", help="accepted for command-line compatibility; nothing is uploaded")
    return p.parse_args(argv)


def _build_stacr_min_config(args):
    """Attribute bag in the protocol runner's vocabulary: a frozen-after-init, quantised, fixed-rank STAC-R."""
    return SimpleNamespace(method="stacr", rank=args.stacr_rank, stacr_rank=args.stacr_rank, stacr_residual_mode=args.stacr_residual_mode,
                           stacr_residual_budget=args.stacr_residual_budget, stacr_warmup_steps=0, stacr_quantize_coefficients=True,
                           stacr_quantize_bits=8, stacr_quantize_residuals=True, stacr_residual_quantize_bits=4, stacr_basis_dtype="float16",
                           stacr_min_features=64, stacr_rank_mode="fixed", quiet=True)


def _maybe_apply_stacr(model, args):
    if not args.enable_stacr:
        return []
    if "bert" not in args.model_name_or_path.lower():
        raise ValueError("--enable_stacr in this protocol supports BERT-family encoders only")
    from ..adaptive import STACRConfig, apply_adaptive_stacr

    names = [n for n, _ in model.named_modules() if n.endswith("output.dense") and "attention" not in n]
    bag = _build_stacr_min_config(args)
    cfg = STACRConfig(rank=bag.rank, residual_budget=bag.stacr_residual_budget, residual_mode=bag.stacr_residual_mode,
                      quantize_coefficients=True, quantize_bits=8, quantize_residuals=True, residual_quantize_bits=4)
    return apply_adaptive_stacr(model, cfg, surface="none", target_names=names, min_features=bag.stacr_min_features, allow_empty=True)


def _data(args, vocab, labels):
    from ..datasets import synthetic_token_examples

    def stack(examples, bs):
        return [{k: torch.stack([torch.as_tensor(e[k]) for e in examples[i:i + bs]]) for k in examples[0]} for i in range(0, len(examples), bs)]

    train = synthetic_token_examples(args.train_examples, args.max_length, vocab, args.seed, task="sequence_classification")
    val = synthetic_token_examples(args.eval_examples, args.max_length, vocab, args.seed + 1, task="sequence_classification")
    for ex in train + val:                                   # a learnable rule so that accuracy means something
        ex["labels"] = (ex["input_ids"][:8].sum() % max(labels, 2)).long()
    return stack(train, args.per_device_train_batch_size), stack(val, args.per_device_eval_batch_size)


def _optimizer(model, args):
    if not args.enable_low_rank:
        return torch.optim.AdamW(model.parameters(), lr=args.learning_rate, weight_decay=args.weight_decay), "adamw"
    from .lowrank_optim import GaLoreAdamW, SubTrackAdamW, split_param_groups

    extra = dict(rank=args.lora_r, update_proj_gap=args.subspace_update_interval, scale=args.low_rank_scale, proj_type=args.proj_type)
    if args.low_rank_method == "subtrack":
        extra.update(step_size=args.st_init_step_size, track_interval=max(1, args.subspace_update_interval // 20))
    groups = split_param_groups(model, ["attention", "intermediate", "output"], args.weight_decay, **extra)
    cls = SubTrackAdamW if args.low_rank_method == "subtrack" else GaLoreAdamW
    return cls(groups, lr=args.learning_rate), args.low_rank_method


def _lr_at(step, total, args):
    if step < args.num_warmup_steps:
        return (step + 1) / max(1, args.num_warmup_steps)
    frac = (step - args.num_warmup_steps) / max(1, total - args.num_warmup_steps)
    return {"linear": max(0.0, 1.0 - frac), "cosine": 0.5 * (1 + math.cos(math.pi * min(frac, 1.0))), "constant": 1.0}[args.lr_scheduler_type]


def main(argv=None, sweep_config=None) -> dict:
    import stacr_b200 as S

    from ..models import build_model
    from ..utils import set_seed

    args = parse_args(argv)
    for key, value in (sweep_config or {}).items():
        setattr(args, key, value)
    if args.enable_stacr and "bert" not in args.model_name_or_path.lower():
        raise ValueError("--enable_stacr in this protocol supports BERT-family encoders only")
    set_seed(args.seed)
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    labels = GLUE_LABELS[args.task_name]
    overrides = json.loads(args.model_overrides) if args.model_overrides else {}
    model = build_model(args.model_name_or_path, task="sequence_classification", num_labels=max(labels, 2), **overrides).to(device)
    layers = _maybe_apply_stacr(model, args)
    train, val = _data(args, int(model.config.vocab_size), labels)
    opt, opt_name = _optimizer(model, args)
    accum = max(1, args.gradient_accumulation_steps)
    total = args.max_train_steps or (args.num_train_epochs * math.ceil(len(train) / accum))
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    model.train()
    started, losses, micro = time.perf_counter(), [], 0
    for step in range(total):
        for g in opt.param_groups:
            g["lr"] = args.learning_rate * _lr_at(step, total, args)
        S.set_step([l for l in layers if isinstance(l, S.STACRLinear)], step)
        opt.zero_grad(set_to_none=True)
        value = 0.0
        for _ in range(accum):
            batch = {k: v.to(device) for k, v in train[micro % len(train)].items()}
            micro += 1
            loss = model(**batch).loss / accum
            loss.backward()
            value += float(loss.detach())
        opt.step()
        losses.append(value)
    wall = time.perf_counter() - started
    model.eval()
    hit = seen = 0
    eval_loss = 0.0
    with torch.no_grad():
        for batch in val:
            batch = {k: v.to(device) for k, v in batch.items()}
            out = model(**batch)
            hit += int((out.logits.argmax(-1) == batch["labels"]).sum())
            seen += batch["labels"].numel()
            eval_loss += float(out.loss) * batch["labels"].numel()
    result = {
        "task": args.task_name, "model": args.model_name_or_path, "optimizer": opt_name, "low_rank": bool(args.enable_low_rank),
        "optimizer_rank": args.lora_r if args.enable_low_rank else None, "stacr": bool(args.enable_stacr), "stacr_layers": len(layers),
        "steps": total, "train_loss_first": losses[0] if losses else None, "train_loss_last": losses[-1] if losses else None,
        "eval_accuracy": hit / max(seen, 1), "eval_loss": eval_loss / max(seen, 1), "train_runtime_s": wall,
        "train_samples_per_second": total * accum * args.per_device_train_batch_size / wall if wall > 0 else None,
        "peak_allocated_gib": torch.cuda.max_memory_allocated(device) / 2 ** 30 if device.type == "cuda" else None,
        "optimizer_state_bytes": sum(t.numel() * t.element_size() for st in opt.state.values() for t in st.values() if torch.is_tensor(t)),
        "data": "synthetic",
    }
    if args.output_dir:
        os.makedirs(args.output_dir, exist_ok=True)
        with open(os.path.join(args.output_dir, "all_results.json"), "w") as fh:
            json.dump(result, fh, indent=2)
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
