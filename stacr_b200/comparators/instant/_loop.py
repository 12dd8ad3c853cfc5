"""Shared training loop of the two INSTANT scripts: periodic calibration, AdamW steps, JSON result."""

from __future__ import annotations

import json
import math
import os
import time

import torch

from .callback import Calibrator
from .custom_op import InstantLinear, register_filter
from .model import convert_conv1d_to_linear, freeze_layers, get_svd_layers
from .utils import log_svd_shapes, set_train_seed


def _collate(examples, device):
    return {k: torch.stack([torch.as_tensor(e[k]) for e in examples]).to(device) for k in examples[0]}


def _loss(model, batch):
    out = model(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"), labels=batch["labels"])
    return out.loss if hasattr(out, "loss") else out[0]


def run(args, model, train, val, *, task: str) -> dict:
    device = torch.device(args.device if getattr(args, "device", None) else ("cuda" if torch.cuda.is_available() else "cpu"))
    set_train_seed(args.seed)
    os.makedirs(args.output_dir, exist_ok=True)
    model = convert_conv1d_to_linear(model).to(device)
    freeze_layers(model, args.n_last_layers, args.model_name)
    names = []
    if args.compress:
        names = get_svd_layers(model, model_name=args.model_name)
        register_filter(model, names)
    calib = Calibrator(model, names, var=args.var, over_sampling=args.over_sampling) if names else None
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=args.learning_rate)
    bs = args.batch_size
    batches = [train[i:i + bs] for i in range(0, len(train) - bs + 1, bs)] or [train]
    per_epoch = len(batches)
    total = args.max_steps if args.max_steps and args.max_steps > 0 else per_epoch * max(int(args.epochs), 1)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    started, losses, widths = time.perf_counter(), [], {}
    model.train()
    for step in range(total):
        if calib is not None and step % max(int(args.calib_iter), 1) == 0:
            picks = [batches[(step + j) % per_epoch] for j in range(max(int(args.calib_batches), 1))]
            pieces = []
            for group in picks:                              # optional split of each calibration batch
                size = max(len(group) // max(int(args.num_split), 1), 1)
                pieces += [group[i:i + size] for i in range(0, len(group), size)]
            widths = calib.run((_collate(g, device) for g in pieces), _loss)
            log_svd_shapes(step, calib.P, os.path.join(args.output_dir, "svd_shapes.json"))
        batch = _collate(batches[step % per_epoch], device)
        opt.zero_grad(set_to_none=True)
        loss = _loss(model, batch)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    model.eval()
    val_loss, correct, count = 0.0, 0, 0
    with torch.no_grad():
        for i in range(0, len(val), bs):
            batch = _collate(val[i:i + bs], device)
            out = model(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"), labels=batch["labels"])
            n = batch["input_ids"].shape[0]
            val_loss += float(out.loss) * n
            count += n
            if task == "classification":
                correct += int((out.logits.argmax(-1) == batch["labels"]).sum())
    val_loss /= max(count, 1)
    tokens = train[0]["input_ids"].shape[-1]
    kept = [m.saved_rows(tokens) for m in model.modules() if isinstance(m, InstantLinear)]
    result = {
        "method": "instant" if args.compress else "dense", "model": args.model_name, "steps": total, "seed": args.seed,
        "train_loss_first": losses[0] if losses else None, "train_loss_last": losses[-1] if losses else None,
        "val_loss": val_loss, "compressed_layers": len(names),
        "mean_saved_row_fraction": (sum(kept) / (len(kept) * tokens)) if kept else 1.0,
        "subspace_widths": {k: list(v) for k, v in list(widths.items())[:8]},
        "wall_s": time.perf_counter() - started,
        "peak_alloc_mb": torch.cuda.max_memory_allocated(device) / 2 ** 20 if device.type == "cuda" else None,
    }
    if task == "classification":
        result["val_accuracy"] = correct / max(count, 1)
    else:
        result["val_ppl"] = math.exp(min(val_loss, 50.0))
    with open(os.path.join(args.output_dir, "result.json"), "w") as fh:
        json.dump(result, fh, indent=2)
    return result
