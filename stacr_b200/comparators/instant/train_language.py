"""INSTANT on a GPT-2 family model, WikiText-103 shaped data (parity: comparators/instant/train_language.py).

    python -m stacr_b200.comparators.instant.train_language --model_name gpt2 --compress --max-steps 20 --synthetic
"""

from __future__ import annotations

import argparse


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="INSTANT comparator, causal language modelling")
    p.add_argument("--model_name", default="gpt2", choices=["gpt2", "gpt2-medium", "gpt2-large", "gpt2-xl"])
    p.add_argument("--n-last-layers", type=int, default=0, help="train only the last N blocks (0 = all)")
    p.add_argument("--num_split", type=int, default=1, help="pieces each calibration batch is split into")
    p.add_argument("--calib_batches", type=int, default=5)
    p.add_argument("--calib_iter", type=int, default=50, help="steps between re-calibrations")
    p.add_argument("--output_dir", default="runs-gpt2")
    p.add_argument("--batch-size", type=int, default=4)
    p.add_argument("--learning-rate", type=float, default=2e-5)
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--max-length", type=int, default=512)
    p.add_argument("--max-steps", type=int, default=-1)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--var", type=float, default=0.95, help="energy kept by the subspace")
    p.add_argument("--over_sampling", type=int, default=15)
    p.add_argument("--compress", action="store_true")
    p.add_argument("--dataset", default="wikitext103")
    p.add_argument("--synthetic", action="store_true", help="random tokens instead of the cached corpus")
    p.add_argument("--device", default=None)
    p.add_argument("--model-overrides", default=None, help="JSON of architecture overrides, e.g. a smaller depth")
    return p.parse_args(argv)


def main(argv=None) -> dict:
    import json

    from ...models import build_model
    from . import _loop
    from .dataset_prep import load_wikitext103

    args = parse_args(argv)
    overrides = json.loads(args.model_overrides) if args.model_overrides else {}
    model = build_model(args.model_name, **overrides)
    vocab = int(getattr(model.config, "vocab_size", 50257))
    train, val = load_wikitext103(None, args.max_length, synthetic=True, vocab_size=vocab, seed=args.seed) if args.synthetic \
        else _cached_or_synthetic(args, vocab)
    result = _loop.run(args, model, train, val, task="language")
    print(json.dumps(result))
    return result


def _cached_or_synthetic(args, vocab):
    from .dataset_prep import load_wikitext103

    tokenizer = None
    try:
        from transformers import AutoTokenizer

        tokenizer = AutoTokenizer.from_pretrained(args.model_name, local_files_only=True)
    except Exception:
        pass
    return load_wikitext103(tokenizer, args.max_length, vocab_size=vocab, seed=args.seed)


if __name__ == "__main__":
    main()
