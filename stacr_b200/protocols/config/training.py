"""Protocol configuration dataclasses (parity: stacr/protocols/config/training.py:15-150 of the reference project)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional


@dataclass
class OptimizerConfig:
    name: str = "adamw"
    lr: float = 5e-5
    weight_decay: float = 0.01
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    use_8bit: bool = False
    min_8bit_size: int = 4096

    def get_optimizer_kwargs(self) -> Dict[str, Any]:
        kw = {"lr": self.lr, "weight_decay": self.weight_decay, "betas": tuple(self.betas), "eps": self.eps}
        if self.use_8bit:
            kw["min_8bit_size"] = self.min_8bit_size
        return kw


@dataclass
class TrainingConfig:
    batch_size: int = 8
    seq_len: int = 1024
    max_steps: int = 1000
    gradient_accumulation_steps: int = 1
    warmup_ratio: float = 0.1
    max_grad_norm: Optional[float] = 1.0
    seed: int = 42
    log_every: int = 10
    eval_every: int = 0
    save_every_n_steps: int = 0
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)

    def __post_init__(self):
        if self.batch_size < 1 or self.gradient_accumulation_steps < 1 or self.max_steps < 1:
            raise ValueError("batch_size, gradient_accumulation_steps and max_steps must be positive")
        if not 0 <= self.warmup_ratio <= 1:
            raise ValueError("warmup_ratio must be in [0, 1]")


@dataclass
class BaselineConfig:
    """Which memory baselines are composed with a run."""

    amp: str = "none"                 # none | auto | bf16 | fp16
    checkpointing: str = "none"       # none | auto | transformer_hf | vision_stage | vision_block | attention_only
    offload: str = "none"             # none | cpu | cpu_pinned
    offload_min_bytes: int = 1_000_000
    optimizer_8bit: bool = False
    data_parallel: str = "none"       # none | dp | ddp
    c1_checkpoint_compression: bool = False

    def get_description(self) -> str:
        parts = []
        if self.amp != "none":
            parts.append(f"amp={self.amp}")
        if self.checkpointing != "none":
            parts.append(f"ckpt={self.checkpointing}")
        if self.offload != "none":
            parts.append(f"offload={self.offload}")
        if self.optimizer_8bit:
            parts.append("opt8bit")
        if self.data_parallel != "none":
            parts.append(self.data_parallel)
        if self.c1_checkpoint_compression:
            parts.append("c1")
        return "+".join(parts) if parts else "none"

    def is_default(self) -> bool:
        return self == BaselineConfig()

    @classmethod
    def from_legacy(cls, baseline_str: str) -> "BaselineConfig":
        """Parse strings such as ``"amp+ckpt"`` or ``"bf16+8bit+offload"``."""
        cfg = cls()
        for token in filter(None, (t.strip().lower() for t in str(baseline_str or "").replace(",", "+").split("+"))):
            if token in ("amp", "auto"):
                cfg.amp = "auto"
            elif token in ("bf16", "fp16"):
                cfg.amp = token
            elif token in ("ckpt", "checkpoint", "checkpointing"):
                cfg.checkpointing = "auto"
            elif token in ("offload", "cpu"):
                cfg.offload = "cpu"
            elif token in ("cpu_pinned", "pinned"):
                cfg.offload = "cpu_pinned"
            elif token in ("8bit", "opt8bit", "bnb"):
                cfg.optimizer_8bit = True
            elif token in ("dp", "ddp"):
                cfg.data_parallel = token
            elif token == "c1":
                cfg.c1_checkpoint_compression = True
            elif token not in ("none", "baseline"):
                raise ValueError(f"Unknown baseline token: {token!r}")
        return cfg
