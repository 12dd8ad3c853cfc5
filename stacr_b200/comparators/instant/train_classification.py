"""INSTANT on a BERT-family classifier (parity: comparators/instant/train_classification.py).

    python -m stacr_b200.comparators.instant.train_classification --compress --max-steps 20
"""

from __future__ import annotations

import argparse


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="INSTANT comparator, sequence classification")
    p.add_argument("--n-last-layers", type=int, default=0)
    p.add_argument("--num_split", type=int, default=1)
    p.add_argument("--calib_batches", type=int, default=5)
    p.add_argument("--calib_iter", type=int, default=50)
    p.add_argument("--dataset", default="sst2")
    p.add_argument("--model_name", default="bert-base-uncased")
    p.add_argument("--output_dir", default="runs-main")
    p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--learning-rate", type=float, default=2e-5)
    p.add_argument("--epochs", type=int, default=10)
    p.add_argument("--max-length", type=int, default=512)
    p.add_argument("--max-steps", type=int, default=-1)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--var", type=float, default=0.95)
    p.add_argument("--over_sampling", type=int, default=7)
    p.add_argument("--compress", action="store_true")
    p.add_argument("--device", default=None)
    p.add_argument("--model-overrides", default=None)
    return p.parse_args(argv)


def main(argv=None) -> dict:
    import json

    from ...models import build_model
    from . import _loop
    from .dataset_prep import load_classification

    args = parse_args(argv)
    overrides = json.loads(args.model_overrides) if args.model_overrides else {}
    model = build_model(args.model_name, task="sequence_classification", **overrides)
    vocab = int(getattr(model.config, "vocab_size", 30522))
    train, val = load_classification(args.dataset, None, args.max_length, vocab_size=vocab, seed=args.seed)
    result = _loop.run(args, model, train, val, task="classification")
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
