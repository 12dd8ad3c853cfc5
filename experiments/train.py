"""Run one training configuration (a YAML/JSON file or a named profile) and write its result row as CSV.

    python experiments/train.py --config configs/synthetic_stacr.yaml --output outputs/result.csv --steps 20

Parity: experiments/train.py (``--config``, ``--output``, ``--steps`` -> ``run_config`` -> ``write_csv``).
"""

from __future__ import annotations

try:
    from . import _bootstrap  # noqa: F401
except ImportError:  # run by path
    import _bootstrap  # noqa: F401

import argparse
from pathlib import Path


def main(argv=None) -> dict:
    from stacr_b200.training import run_config
    from stacr_b200.utils import load_yaml, write_csv

    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config", required=True, help="path of a YAML/JSON configuration, or the name of one under configs/")
    parser.add_argument("--output", default="outputs/result.csv")
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--device", default=None)
    args = parser.parse_args(argv)
    path = Path(args.config)
    if not path.exists():
        for suffix in (".yaml", ".yml", ".json"):
            guess = _bootstrap.ROOT / "configs" / f"{args.config}{suffix}"
            if guess.exists():
                path = guess
                break
    cfg = load_yaml(path)
    if args.steps is not None:
        cfg["steps"] = args.steps
    if args.device:
        cfg["device"] = args.device
    row = run_config(cfg)
    write_csv(args.output, [row])
    print(row)
    return row


if __name__ == "__main__":
    main()
