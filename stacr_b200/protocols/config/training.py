"""Protocol configuration dataclasses (parity: stacr/protocols/config/training.py:15-150 of the reference project)."""

from __future__ import annotations

from dataclasses import dataclass, field, fields
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
    """Which memory baselines are composed with a run (they combine: checkpointing + amp + 8-bit optimizer ...).

    ``saved_tensors_offload`` / ``saved_tensors_offload_min_bytes`` are accepted as constructor aliases of ``offload`` /
    ``offload_min_bytes``.
    """

    name: str = "baseline"
    amp: str = "none"                 # none | auto | bf16 | fp16
    amp_dtype: str = "float16"        # dtype "auto" falls back to when bf16 is not supported
    checkpointing: str = "none"       # none | auto | transformer_hf | vision_stage | vision_block | attention_only
    checkpoint_segments: int = 2
    grad_accum_steps: int = 1
    offload: str = "none"             # none | cpu | cpu_pinned
    offload_min_bytes: int = 1_000_000
    optimizer_8bit: bool = False
    data_parallel: str = "none"       # none | dp | ddp
    c1_checkpoint_compression: bool = False
    actnn: str = "none"               # none | L0..L5 (optional package)
    gact: str = "none"                # none | L0..L4 (optional package)
    torchao: str = "none"             # none | auto | adamw8bit | adamw4bit | float8 (optional package)
    galore: str = "none"              # none | "rank=256,update_gap=200,scale=0.25"
    galore_target_modules: str = "none"

    def __post_init__(self):
        if self.grad_accum_steps < 1 or self.checkpoint_segments < 1:
            raise ValueError("grad_accum_steps and checkpoint_segments must be positive")

    @property
    def saved_tensors_offload(self) -> str:
        return self.offload

    @property
    def saved_tensors_offload_min_bytes(self) -> int:
        return self.offload_min_bytes

    def galore_options(self) -> Optional[Dict[str, Any]]:
        """``"rank=256,update_gap=200,scale=0.25"`` -> keyword arguments of the GaLore optimizer factory."""
        if self.galore in ("none", "", None):
            return None
        names = {"rank": ("rank", int), "update_gap": ("update_proj_gap", int), "update_proj_gap": ("update_proj_gap", int),
                 "scale": ("scale", float), "proj_type": ("proj_type", str)}
        out: Dict[str, Any] = {}
        for item in str(self.galore).split(","):
            key, sep, value = item.strip().partition("=")
            if not sep or key not in names:
                raise ValueError(f"Bad galore option {item!r}")
            target, cast = names[key]
            out[target] = cast(value)
        if self.galore_target_modules not in ("none", "", None):
            out["target_modules"] = [t.strip() for t in str(self.galore_target_modules).split(",") if t.strip()]
        return out

    def get_description(self) -> str:
        parts = []
        if self.amp != "none":
            parts.append(f"amp={self.amp}")
        if self.checkpointing != "none":
            parts.append(f"ckpt={self.checkpointing}")
        if self.grad_accum_steps > 1:
            parts.append(f"accum={self.grad_accum_steps}")
        if self.offload != "none":
            parts.append(f"offload={self.offload}")
        if self.optimizer_8bit:
            parts.append("opt8bit")
        if self.data_parallel != "none":
            parts.append(self.data_parallel)
        if self.c1_checkpoint_compression:
            parts.append("c1")
        for key in ("actnn", "gact", "torchao", "galore"):
            if getattr(self, key) != "none":
                parts.append(f"{key}={getattr(self, key)}")
        if self.galore_target_modules not in ("none", "", None):
            parts.append(f"galore_targets={self.galore_target_modules}")
        return "+".join(parts) if parts else "none"

    def is_default(self) -> bool:
        return self == BaselineConfig(name=self.name)

    @classmethod
    def from_mapping(cls, raw: Dict[str, Any]) -> "BaselineConfig":
        alias = {"saved_tensors_offload": "offload", "saved_tensors_offload_min_bytes": "offload_min_bytes"}
        known = {f.name for f in fields(cls)}
        mapped = {alias.get(k, k): v for k, v in raw.items()}
        stray = sorted(set(mapped) - known)
        if stray:
            raise ValueError(f"Unknown baseline options: {stray}")
        return cls(**mapped)

    @classmethod
    def from_legacy(cls, baseline_str: str) -> "BaselineConfig":
        """A single baseline name (``"checkpointing"``, ``"galore"`` ...) or a ``+``-joined list such as ``"bf16+8bit+offload"``."""
        single = {"checkpointing": dict(checkpointing="transformer_hf"), "grad_accum": dict(grad_accum_steps=2), "actnn": dict(actnn="L2"),
                  "gact": dict(gact="L1"), "torchao": dict(torchao="auto"), "galore": dict(galore="rank=128,update_gap=200,scale=0.25")}
        text = str(baseline_str or "").strip().lower()
        if text in single:
            return cls(**single[text])
        cfg = cls()
        for token in filter(None, (t.strip() for t in text.replace(",", "+").split("+"))):
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
            elif token in single:
                for k, v in single[token].items():
                    setattr(cfg, k, v)
            elif token not in ("none", "baseline"):
                raise ValueError(f"Unknown baseline token: {token!r}")
        return cfg
