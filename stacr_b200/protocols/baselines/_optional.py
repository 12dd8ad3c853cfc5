"""Shared machinery of the graceful-skip adapters: a status enum, a result record and an import probe."""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, Optional, Tuple


class AdapterStatus(Enum):
    OK = "ok"
    SKIPPED_NOT_INSTALLED = "skipped_not_installed"
    SKIPPED_INCOMPATIBLE = "skipped_incompatible"
    SKIPPED_NO_CUDA = "skipped_no_cuda"
    ERROR = "error"


@dataclass
class AdapterResult:
    status: AdapterStatus
    message: str = ""
    version: Optional[str] = None
    details: Dict[str, Any] = field(default_factory=dict)

    @property
    def ok(self) -> bool:
        return self.status is AdapterStatus.OK

    @property
    def reason(self) -> str:
        """The message, under the name result records of the optional baselines use."""
        return self.message

    @property
    def meta(self) -> Dict[str, Any]:
        return {"version": self.version, **self.details}

    def to_dict(self) -> Dict[str, Any]:
        return {"status": self.status.value, "message": self.message, "version": self.version, "ok": self.ok, **self.details}


def probe(module_name: str) -> Tuple[bool, Optional[str], Any]:
    """``(available, version-or-error, module)`` without raising."""
    try:
        mod = importlib.import_module(module_name)
        return True, getattr(mod, "__version__", "unknown"), mod
    except Exception as exc:  # noqa: BLE001
        return False, f"{type(exc).__name__}: {exc}", None


def final_json(baseline: str, result: AdapterResult, output_dir: str) -> Dict[str, Any]:
    """The ``final.json`` body of a run whose optional baseline was enabled, skipped or failed.

    A skipped baseline still gets a well-formed record so that sweeps stay complete and plottable.
    """
    return {"baseline": baseline, "status": result.status.value, "reason": result.message, "meta": result.meta, "output_dir": str(output_dir)}
