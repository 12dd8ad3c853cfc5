"""8-bit optimizer factory.

The reference builds ``bitsandbytes`` optimizers here (stacr/protocols/baselines/bnb_optimizer.py:61-176
there) and reports a ``SKIPPED_*`` status when the library is missing.  This framework ships its own block-wise
8-bit AdamW, so ``try_create_8bit_optimizer`` first tries the in-tree kernel-backed optimizer and uses
``bitsandbytes`` only when it is explicitly requested and importable.
"""

from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn


class BNBStatus(Enum):
    OK = "ok"
    OK_INTREE = "ok_intree"
    SKIPPED_NOT_INSTALLED = "skipped_not_installed"
    SKIPPED_NO_CUDA = "skipped_no_cuda"
    SKIPPED_UNSUPPORTED_OPTIMIZER = "skipped_unsupported_optimizer"
    ERROR = "error"


@dataclass
class BNBResult:
    status: BNBStatus
    optimizer: Optional[torch.optim.Optimizer] = None
    message: str = ""
    backend: str = "none"

    @property
    def ok(self) -> bool:
        return self.status in (BNBStatus.OK, BNBStatus.OK_INTREE)

    def to_dict(self) -> Dict[str, Any]:
        return {"status": self.status.value, "message": self.message, "backend": self.backend, "ok": self.ok}


def check_bnb_available() -> Tuple[bool, Optional[str]]:
    try:
        import bitsandbytes as bnb  # noqa: F401

        return True, getattr(bnb, "__version__", "unknown")
    except Exception as exc:  # noqa: BLE001
        return False, f"{type(exc).__name__}: {exc}"


def try_create_8bit_optimizer(params, optimizer_name: str = "adamw", lr: float = 5e-5, weight_decay: float = 0.01,
                              betas=(0.9, 0.999), eps: float = 1e-8, min_8bit_size: int = 4096, prefer: str = "intree") -> BNBResult:
    name = optimizer_name.lower()
    params = list(params)
    if prefer == "bnb":
        ok, info = check_bnb_available()
        if not ok:
            return BNBResult(BNBStatus.SKIPPED_NOT_INSTALLED, message=str(info))
        if not all(p.is_cuda for p in params):
            return BNBResult(BNBStatus.SKIPPED_NO_CUDA, message="bitsandbytes optimizers need CUDA parameters")
        import bitsandbytes as bnb

        table = {"adamw": "AdamW8bit", "adam": "Adam8bit", "sgd": "SGD8bit"}
        if name not in table:
            return BNBResult(BNBStatus.SKIPPED_UNSUPPORTED_OPTIMIZER, message=name)
        try:
            cls = getattr(bnb.optim, table[name])
            kw = dict(lr=lr, weight_decay=weight_decay)
            if name != "sgd":
                kw.update(betas=betas, eps=eps)
            try:
                opt = cls(params, min_8bit_size=min_8bit_size, **kw)
            except TypeError:  # older releases do not take min_8bit_size
                opt = cls(params, **kw)
            return BNBResult(BNBStatus.OK, opt, backend="bitsandbytes")
        except Exception as exc:  # noqa: BLE001
            return BNBResult(BNBStatus.ERROR, message=f"{type(exc).__name__}: {exc}")
    if name not in ("adamw", "adam"):
        return BNBResult(BNBStatus.SKIPPED_UNSUPPORTED_OPTIMIZER, message=f"in-tree 8-bit optimizer implements AdamW, not {name}")
    from ...optim import AdamW8bit

    opt = AdamW8bit(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay if name == "adamw" else 0.0, min_8bit_size=min_8bit_size)
    return BNBResult(BNBStatus.OK_INTREE, opt, backend="stacr_b200.optim.AdamW8bit")


def estimate_optimizer_savings(model: nn.Module, *, min_8bit_size: int = 4096) -> Dict[str, float]:
    """Bytes of Adam state in fp32 versus block-wise 8-bit (1 byte per moment + 4 bytes per 256-element block)."""
    fp32 = eight = 0
    for p in model.parameters():
        if not p.requires_grad:
            continue
        n = p.numel()
        fp32 += 8 * n
        eight += 8 * n if n < min_8bit_size else 2 * n + 2 * 4 * ((n + 255) // 256)
    return {"fp32_state_bytes": float(fp32), "int8_state_bytes": float(eight), "savings_bytes": float(fp32 - eight),
            "savings_ratio": fp32 / eight if eight else 1.0}
