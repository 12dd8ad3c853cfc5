"""One activation through the tracked compressor and through an untracked random subspace: cosine and relative MSE of each.

Parity: experiments/mechanism_replay.py.
"""

from __future__ import annotations

try:
    from . import _bootstrap  # noqa: F401
except ImportError:
    import _bootstrap  # noqa: F401

import argparse


def main(argv=None) -> dict:
    import torch

    from stacr_b200.comparators.prac import PRACCompressor, PRACConfig
    from stacr_b200.compressor import STACRCompressor, STACRConfig
    from stacr_b200.metrics import cosine_similarity, relative_mse

    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--rank", type=int, default=8)
    parser.add_argument("--rows", type=int, default=64)
    parser.add_argument("--features", type=int, default=512)
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args(argv)
    x = torch.randn(args.rows, args.features, generator=torch.Generator().manual_seed(args.seed))
    tracked = STACRCompressor(STACRConfig(rank=args.rank, residual_budget=0.01, min_features=1, min_numel=1))
    x_tracked = tracked.unpack(tracked.pack(x))
    x_random = PRACCompressor(PRACConfig(rank=args.rank)).reconstruct(x)
    report = {"stacr_cosine": float(cosine_similarity(x, x_tracked)), "stacr_relative_mse": float(relative_mse(x, x_tracked)),
              "prac_cosine": float(cosine_similarity(x, x_random)), "prac_relative_mse": float(relative_mse(x, x_random))}
    print(report)
    return report


if __name__ == "__main__":
    main()
