"""Reconstruction error and stored size of per-batch factorisations (SVD, Tucker-like, TT-like) on one random activation.

Parity: experiments/factorization_benchmark.py.
"""

from __future__ import annotations

try:
    from . import _bootstrap  # noqa: F401
except ImportError:
    import _bootstrap  # noqa: F401

import argparse


def main(argv=None) -> list:
    import torch

    from stacr_b200.comparators.per_batch_factors import factorization_benchmark

    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rank", type=int, default=8)
    parser.add_argument("--rows", type=int, default=64)
    parser.add_argument("--features", type=int, default=512)
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args(argv)
    x = torch.randn(args.rows, args.features, generator=torch.Generator().manual_seed(args.seed))
    rows = factorization_benchmark(x, rank=args.rank)
    for row in rows:
        print(row)
    return rows


if __name__ == "__main__":
    main()
