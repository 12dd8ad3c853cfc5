"""Render every CSV table of a data folder as a LaTeX ``tabular`` (booktabs rules, all cells escaped).

    python -m scripts.make_tables --input paper_data --output outputs/tables

Parity: scripts/make_tables.py:1-53 of the reference project.
"""

from __future__ import annotations

import argparse
import csv
from pathlib import Path

_LATEX = {"\\": r"\textbackslash{}", "&": r"\&", "%": r"\%", "$": r"\$", "#": r"\#", "_": r"\_", "{": r"\{", "}": r"\}",
          "~": r"\textasciitilde{}", "^": r"\textasciicircum{}"}


def escape_latex(value) -> str:
    return "".join(_LATEX.get(ch, ch) for ch in str(value))


def csv_to_latex(path: Path) -> str:
    with Path(path).open(newline="", encoding="utf-8") as fh:
        rows = list(csv.DictReader(fh))
    if not rows:
        return ""
    cols = list(rows[0])

    def line(cells):
        return " & ".join(escape_latex(c) for c in cells) + r" \\"

    body = [line(row[c] for c in cols) for row in rows]
    return "\n".join([r"\begin{tabular}{" + "l" * len(cols) + "}", r"\toprule", line(cols), r"\midrule", *body, r"\bottomrule", r"\end{tabular}"])


def main(argv=None) -> None:
    from .evidence import default_data_dir

    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--input", default=str(default_data_dir()))
    parser.add_argument("--output", default="outputs/tables")
    args = parser.parse_args(argv)
    out = Path(args.output)
    out.mkdir(parents=True, exist_ok=True)
    for table in sorted(Path(args.input).glob("*.csv")):
        (out / f"{table.stem}.tex").write_text(csv_to_latex(table), encoding="utf-8")


if __name__ == "__main__":
    main()
