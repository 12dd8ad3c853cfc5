"""Concatenate the per-experiment CSV files of an output folder into one table (union of columns).

    python -m scripts.aggregate_results --input outputs --output outputs/main_results.csv

Earlier aggregates (``main_results.csv``, ``demo_results.csv``) and the output file itself are not re-read.
Parity: scripts/aggregate_results.py:1-42 of the reference project.
"""

from __future__ import annotations

import argparse
import csv
from pathlib import Path
from typing import Dict, List, Optional

AGGREGATE_NAMES = frozenset({"main_results.csv", "demo_results.csv"})


def read_rows(folder: Path, exclude: Optional[Path] = None) -> List[Dict[str, str]]:
    skip = exclude.resolve() if exclude is not None else None
    rows: List[Dict[str, str]] = []
    for path in sorted(Path(folder).glob("*.csv")):
        if path.name in AGGREGATE_NAMES or (skip is not None and path.resolve() == skip):
            continue
        with path.open(newline="", encoding="utf-8") as fh:
            rows += [dict(r) for r in csv.DictReader(fh)]
    return rows


def write_rows(path: Path, rows: List[Dict[str, str]]) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    if not rows:
        path.write_text("", encoding="utf-8")
        return
    with path.open("w", newline="", encoding="utf-8") as fh:
        writer = csv.DictWriter(fh, fieldnames=sorted({k for r in rows for k in r}))
        writer.writeheader()
        writer.writerows(rows)


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--input", default="outputs")
    parser.add_argument("--output", default="outputs/main_results.csv")
    args = parser.parse_args(argv)
    out = Path(args.output)
    write_rows(out, read_rows(Path(args.input), exclude=out))


if __name__ == "__main__":
    main()
