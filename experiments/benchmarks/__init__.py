"""Measurement grids (``python -m stacr benchmarks list|run``).

Every grid of ``registry.EXPERIMENTS`` is importable and runnable as ``experiments.benchmarks.<grid>`` (the module path
that result files and papers cite) without a file per grid: a meta-path finder installed here synthesises the module for
any registered grid that has no source file of its own.  Grids with helpers of their own (``lora``, ``peak_anatomy``,
``rate_distortion``, ...) keep a real module, which takes precedence.
"""

from __future__ import annotations

import importlib.abc
import importlib.machinery
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))

# names that callers of the reference project import from particular grid modules, re-exported by the synthesised ones
_EXTRA_SOURCE = {
    "hardware_runtime": "from experiments.benchmarks.probes import gpu_gib  # noqa: F401",
    "basis_storage": "from stacr_b200.comparators.activation import FatFunction, FatLinear, apply_fat  # noqa: F401",
    "single_model_fidelity": "from experiments.benchmarks.probes import grads  # noqa: F401",
    "large_models": "from experiments.benchmarks.probes import maxbatch, maxlen, one, sweep  # noqa: F401",
    "sequence_length": "from experiments.benchmarks.probes import maxbatch, maxlen, one, sweep  # noqa: F401",
    "instant_comparison": "enumerate_cells = cells",
    "subtrack_composition": "enumerate_cells = cells",
}

_SOURCE = '''"""{description}.

Grid ``{grid}`` ({category}; {n_cells} cells), declared in ``experiments.benchmarks.registry``.

    python -m experiments.benchmarks.{grid} --dry-run
    python -m experiments.benchmarks.{grid} --steps 20 --seeds 42
"""
from experiments.benchmarks import _entry
from experiments.benchmarks.probes import complement  # noqa: F401

_entry.bind(globals(), {grid!r})
{extra}

if __name__ == "__main__":
    raise SystemExit(main())
'''


class _GridLoader(importlib.abc.InspectLoader):
    def __init__(self, grid: str):
        self.grid = grid

    def is_package(self, fullname):
        return False

    def get_source(self, fullname):
        from ._entry import describe

        meta = describe(self.grid)
        return _SOURCE.format(grid=self.grid, description=str(meta.get("description", self.grid)).rstrip("."),
                              category=meta.get("category", "grid"), n_cells=meta["n_cells"], extra=_EXTRA_SOURCE.get(self.grid, ""))

    def exec_module(self, module):
        exec(self.get_code(module.__name__), module.__dict__)


class _GridFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        prefix = __name__ + "."
        if not fullname.startswith(prefix):
            return None
        grid = fullname[len(prefix):]
        if "." in grid or grid.startswith("_") or os.path.exists(os.path.join(_HERE, grid + ".py")):
            return None
        from .registry import EXPERIMENTS

        if grid not in EXPERIMENTS:
            return None
        return importlib.machinery.ModuleSpec(fullname, _GridLoader(grid), origin=f"<grid {grid}>")


if not any(isinstance(f, _GridFinder) for f in sys.meta_path):
    sys.meta_path.append(_GridFinder())
