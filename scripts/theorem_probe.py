"""Per-layer checks of the gradient-fidelity bounds on saved checkpoints.

For every MLP/attention projection the probe records the layer input ``A`` (tokens x in) and the output gradient
``G`` (tokens x out) of one batch, forms the exact weight gradient ``g = vec(G^T A)`` and its rank-r version
``g_r = vec(G^T A P)`` with ``P`` the projector on the top-r right singular vectors of ``A``, and reports

* ``EV_A``   fraction of ``||A||_F^2`` kept by ``P``;
* ``p``      ``||g - g_r||^2 / ||g||^2`` and the bound ``cos(g, g_r) >= sqrt(1 - p)`` (stated only for ``p < 1``);
* ``q``      ratio of the gradient gains on signal and residual, ``mu_sig^2 / mu_res^2`` with
             ``mu_sig^2 = ||G^T A P||^2 / ||A P||^2`` and ``mu_res^2 = ||G^T (A - A P)||^2 / ||A - A P||^2``, and
             the bridge ``cos^2 = q EV / (q EV + 1 - EV)``;
* ``kappa_G`` ``||G||_2 ||A||_F / ||G^T A||_F``.

Paired mode (a dense checkpoint and a compressed one) adds, against the compressed model's actual gradient
``g_c``: ``s = ||g - g_c||^2 / ||g||^2``, its cosine and bound, and the cross term ``xi = <g - g_r, g_r - g_c> / ||g||^2``.
The two checkpoints are different trained states, so paired numbers contain trajectory drift as well as
compression error.

    python -m scripts.theorem_probe --checkpoint run/ckpt.pt --model gpt2-tiny --task synthetic
    python -m scripts.theorem_probe --baseline-checkpoint a.pt --stacr-checkpoint b.pt --model bert-tiny --task synthetic

Parity: scripts/theorem_probe.py:1-630 of the reference project (same metric names and output layout); the data
here defaults to seeded synthetic tokens because the image has no dataset cache.
"""

from __future__ import annotations

import argparse
import json
import math
import time
from pathlib import Path
from typing import Dict, Optional

import torch
from torch import nn

TASKS = ("synthetic", "sst2", "mrpc", "wikitext103")
_TARGET_PARENTS = ("mlp", "attention", "attn", "intermediate", "output", "self", "self_attn")


def cosine_bound(squared_relative_error: float) -> Optional[float]:
    """``sqrt(1 - e)``: the sharp lower bound on the cosine, defined only for ``0 <= e < 1``."""
    return math.sqrt(1.0 - squared_relative_error) if 0.0 <= squared_relative_error < 1.0 else None


def finite_json(value):
    """Replace NaN/inf by ``None`` recursively so that the report is strict JSON."""
    if isinstance(value, dict):
        return {k: finite_json(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [finite_json(v) for v in value]
    if isinstance(value, float) and not math.isfinite(value):
        return None
    return value


def _is_projection(module: nn.Module) -> bool:
    return isinstance(module, nn.Linear) or type(module).__name__ in ("Conv1D", "STACRLinear")


def target_names(model: nn.Module):
    names = []
    for name, module in model.named_modules():
        parts = name.split(".")
        if _is_projection(module) and len(parts) >= 2 and (parts[-2] in _TARGET_PARENTS or parts[-1] in ("fc1", "fc2")):
            if not any(name.startswith(n + ".") for n in names):
                names.append(name)
    return names


class LayerRecorder:
    """Forward/backward hooks that keep each target's input, output gradient and weight gradient for one batch."""

    def __init__(self, model: nn.Module):
        self.model, self.inputs, self.out_grads, self.handles = model, {}, {}, []
        self.modules = {n: m for n, m in model.named_modules() if n in set(target_names(model))}
        for name, module in self.modules.items():
            self.handles.append(module.register_forward_hook(self._fwd(name)))
            self.handles.append(module.register_full_backward_hook(self._bwd(name)))

    def _fwd(self, name):
        def hook(_m, args, _out):
            self.inputs[name] = args[0].detach().float().cpu()
        return hook

    def _bwd(self, name):
        def hook(_m, _gin, gout):
            if gout[0] is not None:
                self.out_grads[name] = gout[0].detach().float().cpu()
        return hook

    def run(self, batch: Dict[str, torch.Tensor], device):
        self.model.zero_grad(set_to_none=True)
        out = self.model(**{k: v.to(device) for k, v in batch.items()})
        loss = out.loss if hasattr(out, "loss") else out[0]
        loss.backward()
        weight_grads = {}
        for name, module in self.modules.items():
            w = getattr(module, "weight", None)
            if w is None and hasattr(module, "linear"):
                w = module.linear.weight
            if w is not None and w.grad is not None:
                g = w.grad.detach().float().cpu()
                transposed = type(module).__name__ == "Conv1D" or bool(getattr(module, "transposed", False))
                weight_grads[name] = (g.t() if transposed else g).reshape(-1)
        for h in self.handles:
            h.remove()
        self.model.zero_grad(set_to_none=True)
        return self.inputs, self.out_grads, weight_grads


def projection_metrics(inputs, out_grads, weight_grads, rank: int):
    tensors, report = {}, {}
    for name, a in inputs.items():
        g = out_grads.get(name)
        if g is None or a.dim() not in (2, 3):
            continue
        a2, g2 = a.reshape(-1, a.shape[-1]).float(), g.reshape(-1, g.shape[-1]).float()
        if a2.shape[1] < 2 * rank:
            continue
        grad_true = (g2.t() @ a2)
        gnorm2 = float((grad_true ** 2).sum())
        if gnorm2 < 1e-40:
            continue
        _, _, vh = torch.linalg.svd(a2, full_matrices=False)
        q = vh[:rank].t()
        a_sig = (a2 @ q) @ q.t()
        a_res = a2 - a_sig
        grad_sig, grad_res = g2.t() @ a_sig, g2.t() @ a_res
        total, sig2, res2 = float((a2 ** 2).sum()), float((a_sig ** 2).sum()), float((a_res ** 2).sum())
        ev = 1.0 - res2 / (total + 1e-30)
        p = float((grad_res ** 2).sum()) / gnorm2
        cos_obs = float((grad_true * grad_sig).sum() / (grad_true.norm() * grad_sig.norm() + 1e-30))
        if sig2 > 1e-20 and res2 > 1e-20:
            mu_sig, mu_res = float((grad_sig ** 2).sum()) / sig2, float((grad_res ** 2).sum()) / res2
            gain = mu_sig / (mu_res + 1e-30)
        else:
            mu_sig = mu_res = 0.0
            gain = float("nan")
        bridge = math.sqrt(max(gain * ev / (gain * ev + 1.0 - ev), 0.0)) if gain == gain and gain > 0 else float("nan")
        flat = grad_true.reshape(-1)
        tensors[name] = {"g_true": flat, "g_proj": grad_sig.reshape(-1)}
        report[name] = {
            "rank": rank, "shape": list(a2.shape), "EV_A": ev, "p": p, "q": gain, "mu_sig_sq": mu_sig, "mu_res_sq": mu_res,
            "kappa_G": float(torch.linalg.matrix_norm(g2, ord=2)) * math.sqrt(total) / (math.sqrt(gnorm2) + 1e-30),
            "cos_proj_observed": cos_obs, "cos_proj_bound": cosine_bound(p), "cos_q_bridge": bridge,
            "grad_vector_matches_weight_grad": name in weight_grads and weight_grads[name].shape == flat.shape
            and bool(torch.allclose(flat, weight_grads[name], atol=1e-4, rtol=1e-3)),
        }
    return tensors, report


def pair_metrics(tensors, report, compressed_grads):
    out = {}
    for name, t in tensors.items():
        gc = compressed_grads.get(name)
        if gc is None or gc.shape != t["g_true"].shape:
            continue
        g, gr = t["g_true"], t["g_proj"]
        n2 = float((g ** 2).sum())
        s = float(((g - gc) ** 2).sum()) / n2
        out[name] = {**report[name], "s": s, "xi": float(torch.dot(g - gr, gr - gc)) / n2,
                     "cos_full_observed": float(torch.dot(g, gc) / (g.norm() * gc.norm() + 1e-30)), "cos_full_bound": cosine_bound(s)}
    return out


def aggregate(per_layer: Dict[str, dict]) -> dict:
    if not per_layer:
        return {"num_layers": 0}

    def values(key):
        return [v[key] for v in per_layer.values() if isinstance(v.get(key), (int, float)) and math.isfinite(v[key])]

    def mean(key):
        vals = values(key)
        return sum(vals) / len(vals) if vals else None

    summary = {"num_layers": len(per_layer)}
    for key in ("EV_A", "p", "q", "kappa_G", "cos_proj_observed", "cos_proj_bound", "cos_q_bridge"):
        summary["mean_" + key] = mean(key)
    summary["min_cos_proj_observed"] = min(values("cos_proj_observed"), default=None)
    violations = [n for n, v in per_layer.items() if v.get("cos_proj_bound") is not None and v["cos_proj_observed"] < v["cos_proj_bound"] - 1e-4]
    summary["projection_bound_violations"] = len(violations)
    summary["grad_vectors_match"] = sum(bool(v.get("grad_vector_matches_weight_grad")) for v in per_layer.values())
    if any("cos_full_observed" in v for v in per_layer.values()):
        for key in ("s", "xi", "cos_full_observed", "cos_full_bound"):
            summary["mean_" + key] = mean(key)
        summary["min_cos_full_observed"] = min(values("cos_full_observed"), default=None)
    return summary


def _state_dict(path: str):
    blob = torch.load(path, map_location="cpu", weights_only=False)
    for key in ("model", "model_state_dict", "state_dict"):
        if isinstance(blob, dict) and isinstance(blob.get(key), dict):
            return blob[key]
    return blob


def _task_kind(model_name: str) -> str:
    return "sequence_classification" if "bert" in model_name.lower() else "language_modeling"


def load_plain(model_name: str, path: str, device):
    from stacr_b200.models import build_model

    model = build_model(model_name, _task_kind(model_name))
    model.load_state_dict(_state_dict(path), strict=True)
    return model.to(device).eval()  # eval(): dropout off; gradients still flow


def load_compressed(model_name: str, path: str, device, rank: int, budget: float, mode: str):
    """Rebuild the wrapped model, load weights and bases strictly, and freeze the bases so that the probe reads but never updates them."""
    from stacr_b200 import apply_stacr
    from stacr_b200.models import build_model

    model = build_model(model_name, _task_kind(model_name))
    layers = apply_stacr(model, rank=rank, residual_budget=budget, residual_mode=mode, surface="mlp+attention", min_features=2 * rank,
                         allow_empty=True, turbo_after_step=None, freeze_after_warmup=True, warmup_steps=0)
    state = _state_dict(path)
    missing, unexpected = model.load_state_dict(state, strict=False)
    missing = [k for k in missing if not k.rsplit(".", 1)[-1].startswith("_")]
    if missing or unexpected:
        raise RuntimeError(f"checkpoint does not match the compressed model: missing={missing[:5]} unexpected={list(unexpected)[:5]}")
    model.to(device).train()
    for m in model.modules():
        if isinstance(m, nn.Dropout):
            m.p = 0.0
    for layer in layers:
        layer.set_step(10 ** 6)
    return model


def build_batch(task: str, model, batch_size: int, max_length: int, seed: int):
    if task != "synthetic":
        raise SystemExit(f"task {task!r} needs a local dataset cache, which this environment does not provide; use --task synthetic")
    from stacr_b200.datasets import synthetic_token_examples

    cfg = getattr(model, "config", None)
    vocab = int(getattr(cfg, "vocab_size", 1000))
    seq = min(max_length, int(getattr(cfg, "n_positions", getattr(cfg, "max_position_embeddings", max_length))))
    kind = "sequence_classification" if type(model).__name__.endswith("SequenceClassification") else "language_modeling"
    examples = synthetic_token_examples(batch_size, seq, vocab, seed, kind)
    return {k: torch.stack([torch.as_tensor(e[k]) for e in examples]) for k in examples[0]}


def main(argv=None) -> dict:
    parser = argparse.ArgumentParser(description="Gradient-bound probe on saved checkpoints")
    parser.add_argument("--checkpoint", help="single checkpoint: projection probe at that state")
    parser.add_argument("--baseline-checkpoint", help="dense checkpoint of a pair")
    parser.add_argument("--stacr-checkpoint", help="compressed checkpoint of a pair")
    parser.add_argument("--task", default="synthetic", choices=TASKS)
    parser.add_argument("--model", default="bert-tiny")
    parser.add_argument("--rank", type=int, default=8)
    parser.add_argument("--max-length", type=int, default=128)
    parser.add_argument("--batch-size", type=int, default=32)
    parser.add_argument("--seed", type=int, default=42)
    parser.add_argument("--stacr-residual-budget", type=float, default=0.005)
    parser.add_argument("--stacr-residual-mode", default="block_sparse")
    parser.add_argument("--output")
    args = parser.parse_args(argv)
    if min(args.rank, args.batch_size, args.max_length) < 1:
        parser.error("rank, batch-size and max-length must be positive")
    single = args.checkpoint is not None
    pair = args.baseline_checkpoint is not None and args.stacr_checkpoint is not None
    if single and pair:
        raise SystemExit("Use either --checkpoint or the paired --baseline-checkpoint/--stacr-checkpoint form, not both.")
    if not single and not pair:
        raise SystemExit("Provide either --checkpoint or both --baseline-checkpoint and --stacr-checkpoint.")

    torch.manual_seed(args.seed)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    t0 = time.time()
    dense = load_plain(args.model, args.checkpoint if single else args.baseline_checkpoint, device)
    batch = build_batch(args.task, dense, args.batch_size, args.max_length, args.seed)
    inputs, out_grads, wgrads = LayerRecorder(dense).run(batch, device)
    tensors, per_layer = projection_metrics(inputs, out_grads, wgrads, args.rank)
    if pair:
        compressed = load_compressed(args.model, args.stacr_checkpoint, device, args.rank, args.stacr_residual_budget, args.stacr_residual_mode)
        _, _, cgrads = LayerRecorder(compressed).run(batch, device)
        per_layer = pair_metrics(tensors, per_layer, cgrads)
    summary = aggregate(per_layer)
    if not summary["num_layers"]:
        raise RuntimeError("No layers produced valid gradient measurements; check model targets, rank and checkpoint pair")
    report = {
        "mode": "paired" if pair else "single",
        "metadata": {
            "task": args.task, "model": args.model, "rank": args.rank, "seed": args.seed, "probe_time_s": time.time() - t0,
            "checkpoint": args.checkpoint and Path(args.checkpoint).name,
            "baseline_checkpoint": args.baseline_checkpoint and Path(args.baseline_checkpoint).name,
            "stacr_checkpoint": args.stacr_checkpoint and Path(args.stacr_checkpoint).name,
            "comparison_scope": "different_trained_checkpoints" if pair else "same_state_projection",
            "dropout": "disabled", "compression": "enabled with read-only basis and runtime state",
            "batch_size": args.batch_size, "max_length": args.max_length,
        },
        "summary": summary, "per_layer": per_layer,
    }
    print(f"theorem probe: {summary['num_layers']} layers, mode={report['mode']}")
    for key, value in summary.items():
        print(f"  {key}: {'not applicable' if value is None else value}")
    out = Path(args.output) if args.output else Path(args.stacr_checkpoint if pair else args.checkpoint).parent / "theorem_probe.json"
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text(json.dumps(finite_json(report), indent=2, allow_nan=False) + "\n", encoding="utf-8")
    print(f"Saved to {out}")
    return report


if __name__ == "__main__":
    main()
