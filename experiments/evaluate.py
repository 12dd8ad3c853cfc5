"""Print a result CSV as an aligned table, optionally a subset of columns.

    python experiments/evaluate.py --csv outputs/result.csv [--columns loss tokens_per_s]

Parity: experiments/evaluate.py.
"""

from __future__ import annotations

try:
    from . import _bootstrap  # noqa: F401
except ImportError:
    import _bootstrap  # noqa: F401

import argparse


def main(argv=None) -> int:
    import pandas as pd

    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--csv", required=True)
    parser.add_argument("--columns", nargs="*", default=None)
    args = parser.parse_args(argv)
    frame = pd.read_csv(args.csv)
    if args.columns:
        frame = frame[[c for c in args.columns if c in frame.columns]]
    print(frame.to_string(index=False))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
