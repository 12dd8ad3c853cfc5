"""C1: compress the tensor kept at an activation-checkpoint boundary.

A checkpointed transformer block normally keeps its input (``tokens x hidden``) until backward.  C1 keeps
``coefficients = input @ basis`` (optionally int8 with one scale per row) instead, reconstructs
``coefficients @ basis^T`` in backward, replays the block with the RNG state restored and the compression
replay guard set, and back-propagates through the replay.  Both parameter and input gradients become
approximate, which is why the reference reports this as a negative result; it is provided for parity.
Parity: stacr/protocols/checkpointing.py:102-1378 of the reference project (config/spec/record dataclasses,
codec with non-finite dense fallbacks and first-event forensics, site registry and runtime, the custom
checkpoint autograd function, saved-tensor hooks, site discovery for GPT-2 / NeoX-LLaMA / BERT, and the
enable function that rejects tensor- and data-parallel wrappers).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
from torch import nn

from ..adaptive_checkpointing import get_global_recomputation_guard
from ..oja import orthonormalize


@dataclass
class STACRCheckpointConfig:
    enabled: bool = False
    target: str = "decoder_block_input"
    rank: Optional[int] = None
    warmup_steps: int = 500
    residual_mode: str = "none"
    residual_budget: float = 0.005
    refresh_trigger: str = "residual_energy"
    refresh_period: int = 200
    refresh_energy_threshold_mode: str = "auto"
    refresh_energy_threshold: float = 0.15
    min_numel: int = 1 << 20
    basis_dtype: str = "auto"
    quantize_coefficients: bool = False
    quantize_bits: int = 8
    quantize_residuals: bool = True
    residual_quantize_bits: int = 4
    allow_inner_stacr: bool = False
    planner: str = "heuristic"


@dataclass(frozen=True)
class STACRCheckpointSpec:
    site_id: str
    module_type: str
    model_family: str
    hidden_size: int
    rank: int
    residual_mode: str = "none"
    residual_budget: float = 0.0
    basis_dtype: torch.dtype = torch.float32
    quantize_coefficients: bool = False
    quantize_bits: int = 8
    quantize_residuals: bool = False
    residual_quantize_bits: int = 4
    warmup_steps: int = 0
    refresh_trigger: str = "residual_energy"
    refresh_period: int = 200
    refresh_energy_threshold: float = 0.15
    target_arg_index: int = 0
    min_numel: int = 0


@dataclass
class CompressedBoundaryRecord:
    site_id: str
    original_shape: Tuple[int, ...]
    original_dtype: torch.dtype
    device: torch.device
    is_dense_fallback: bool
    dense_tensor: Optional[torch.Tensor] = None
    coeff: Optional[torch.Tensor] = None
    coeff_scale: Optional[torch.Tensor] = None
    coeff_quantized: bool = False
    basis: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class CheckpointSiteCandidate:
    name: str
    module: nn.Module
    model_family: str
    hidden_size: int


def _default_ckpt_rank(model_family: str, hidden_size: int) -> int:
    return max(8, min(hidden_size // 8, 128))


def _resolve_ckpt_basis_dtype(mode: str, amp_mode: str, device: torch.device) -> torch.dtype:
    table = {"float32": torch.float32, "fp32": torch.float32, "float16": torch.float16, "fp16": torch.float16,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    if mode in table:
        return table[mode]
    amp = str(amp_mode).lower()
    if device.type == "cuda" and amp in ("bf16", "auto"):
        return torch.bfloat16
    return torch.float16 if (device.type == "cuda" and amp == "fp16") else torch.float32


def _resolve_ckpt_refresh_energy_threshold(mode: str, value: float, rank: int, hidden: int) -> float:
    if mode != "auto":
        return float(value)
    return float(min(0.5, max(value, 1.0 - rank / max(1, hidden)) * 0.5 + 0.05))


class CheckpointBoundaryCodec(nn.Module):
    """Per-site codec.  State (basis, counters, telemetry) lives in buffers so it is checkpointed with the model."""

    FALLBACK_REASONS = ("input_nonfinite", "basis_nonfinite", "coeff_nonfinite", "scale_nonfinite", "recon_nonfinite", "energy_nonfinite")

    def __init__(self, spec: STACRCheckpointSpec):
        super().__init__()
        self.spec = spec
        self.register_buffer("basis", torch.zeros(spec.hidden_size, spec.rank, dtype=spec.basis_dtype))
        self.register_buffer("_basis_ready", torch.zeros((), dtype=torch.bool))
        self.register_buffer("_steps", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_packs", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_unpacks", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_refreshes", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_raw_bytes", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_stored_bytes", torch.zeros((), dtype=torch.int64))
        self.register_buffer("_last_energy", torch.zeros((), dtype=torch.float32))
        self.fallbacks: Dict[str, int] = {}
        self.first_nonfinite: Optional[Dict[str, Any]] = None
        self.refresh_reasons: Dict[str, int] = {}

    # ------------------------------------------------------------------ counters
    @property
    def pack_count(self) -> int:
        return int(self._packs)

    @property
    def unpack_count(self) -> int:
        return int(self._unpacks)

    @property
    def basis_refresh_count(self) -> int:
        return int(self._refreshes)

    @property
    def step_count(self) -> int:
        return int(self._steps)

    @property
    def basis_initialized(self) -> bool:
        return bool(self._basis_ready)

    # ------------------------------------------------------------------ helpers
    def _flatten(self, t: torch.Tensor) -> torch.Tensor:
        return t.reshape(-1, t.shape[-1])

    def _dense(self, t: torch.Tensor, reason: Optional[str]) -> CompressedBoundaryRecord:
        if reason:
            self.fallbacks[reason] = self.fallbacks.get(reason, 0) + 1
            if self.first_nonfinite is None and reason.endswith("nonfinite"):
                self.first_nonfinite = {"reason": reason, "step": self.step_count, "max_abs": float(t.detach().abs().nan_to_num(posinf=0, neginf=0).max())}
        n = t.numel() * t.element_size()
        self._raw_bytes += n
        self._stored_bytes += n
        return CompressedBoundaryRecord(self.spec.site_id, tuple(t.shape), t.dtype, t.device, True, dense_tensor=t.detach())

    def _compute_basis(self, flat: torch.Tensor) -> torch.Tensor:
        x = flat.detach().float()
        r = self.spec.rank
        if x.shape[0] < r:
            gen = torch.Generator(device="cpu").manual_seed(0)
            return orthonormalize(torch.randn(x.shape[1], r, generator=gen).to(x.device))
        if x.shape[1] > 1024:
            _, _, v = torch.svd_lowrank(x, q=min(x.shape[1], r + 4), niter=2)
            return orthonormalize(v[:, :r].contiguous())
        return orthonormalize(torch.linalg.svd(x, full_matrices=False).Vh[:r].t().contiguous())

    def _update_basis(self, flat: torch.Tensor, *, reason: str) -> None:
        self.basis = self._compute_basis(flat).to(self.spec.basis_dtype)  # rebind
        if bool(self._basis_ready):
            self._refreshes += 1
            self.refresh_reasons[reason] = self.refresh_reasons.get(reason, 0) + 1
        self._basis_ready.fill_(True)

    def _should_refresh(self, energy: float) -> Optional[str]:
        s = self.spec
        since = self.step_count - s.warmup_steps
        if s.refresh_trigger in ("fixed", "hybrid") and since > 0 and since % max(1, s.refresh_period) == 0:
            return "fixed"
        if s.refresh_trigger in ("residual_energy", "hybrid") and energy > s.refresh_energy_threshold:
            return "residual_energy"
        return None

    @staticmethod
    def _on_kernels(flat: torch.Tensor, rank: int) -> bool:
        """bf16 CUDA boundary tensors run the codec on the in-tree kernels: tensor-core projection, reduction kernels for the
        Pythagoras energy, per-row int8 codec, and the low-rank reconstruction kernel on the way back."""
        from ..ops import _lib

        return flat.is_cuda and flat.dtype == torch.bfloat16 and flat.shape[1] % 8 == 0 and rank <= 32 and _lib.available()

    def _project(self, flat: torch.Tensor) -> torch.Tensor:
        if self._on_kernels(flat, self.spec.rank):
            from ..layers import _basis_views
            from ..ops import stacr_ops

            _, qt = _basis_views(self.basis)
            return stacr_ops.project(flat.contiguous(), qt)[:, : self.basis.shape[1]]          # fp32 coefficients
        return flat @ self.basis.to(flat.dtype)

    @staticmethod
    def _sum_squares(t: torch.Tensor) -> torch.Tensor:
        if t.is_cuda and t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous():
            from ..ops import pack_ops

            return pack_ops.sum_squares(t)
        return t.float().square().sum()

    def _quantize_coefficients(self, coeff: torch.Tensor):
        if coeff.is_cuda and coeff.dtype in (torch.float32, torch.bfloat16) and coeff.stride(1) == 1:
            from ..ops import pack_ops

            return pack_ops.quantize_rows_int8(coeff)
        amax = coeff.abs().amax(dim=1, keepdim=True).float()
        scale = (amax / 127.0).clamp_min(torch.finfo(torch.float32).tiny)
        q = torch.round(coeff.float() / scale).clamp_(-127, 127).to(torch.int8)
        return q, scale

    def _dequantize_coefficients(self, q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        return (q.float() * scale).to(dtype)

    # ------------------------------------------------------------------ pack / unpack
    def pack_tensor(self, tensor: torch.Tensor, *, training: bool) -> CompressedBoundaryRecord:
        s = self.spec
        if not training or tensor.numel() < s.min_numel or tensor.shape[-1] != s.hidden_size or not tensor.is_floating_point():
            return self._dense(tensor, None)
        self._packs += 1
        if training:
            self._steps += 1
        if self.step_count <= s.warmup_steps and not self.basis_initialized and s.warmup_steps > 0:
            return self._dense(tensor, "warmup")
        if not torch.isfinite(tensor).all():
            return self._dense(tensor, "input_nonfinite")
        flat = self._flatten(tensor)
        if self.basis.device != flat.device:
            self.basis = self.basis.to(flat.device)
        if not self.basis_initialized:
            self._update_basis(flat, reason="init")
        if not torch.isfinite(self.basis).all():
            return self._dense(tensor, "basis_nonfinite")
        coeff = self._project(flat)
        if not torch.isfinite(coeff).all():
            return self._dense(tensor, "coeff_nonfinite")
        x2, c2 = self._sum_squares(flat), self._sum_squares(coeff if coeff.is_contiguous() else coeff.contiguous())
        energy = float(torch.sqrt((x2 - c2).clamp_min(0)) / (torch.sqrt(x2) + 1e-8))
        if energy != energy:
            return self._dense(tensor, "energy_nonfinite")
        self._last_energy.fill_(energy)
        reason = self._should_refresh(energy)
        if reason is not None:
            self._update_basis(flat, reason=reason)
            coeff = self._project(flat)
        rec = CompressedBoundaryRecord(s.site_id, tuple(tensor.shape), tensor.dtype, tensor.device, False, basis=self.basis)
        if s.quantize_coefficients:
            cq, scale = self._quantize_coefficients(coeff)
            if not torch.isfinite(scale).all():
                return self._dense(tensor, "scale_nonfinite")
            rec.coeff, rec.coeff_scale, rec.coeff_quantized = cq, scale, True
            stored = cq.numel() + scale.numel() * 4
        else:
            rec.coeff = coeff
            stored = coeff.numel() * coeff.element_size()
        self._raw_bytes += tensor.numel() * tensor.element_size()
        self._stored_bytes += stored
        return rec

    def unpack_record(self, packed: CompressedBoundaryRecord) -> torch.Tensor:
        self._unpacks += 1
        if packed.is_dense_fallback:
            return packed.dense_tensor
        hidden = packed.basis.shape[0]
        if packed.coeff.is_cuda and packed.original_dtype == torch.bfloat16 and hidden % 8 == 0 and packed.basis.shape[1] <= 32:
            from ..ops import pack_ops, stacr_ops

            # dequantise and rebuild C Q^T with the reconstruction kernel of the compressed layers (bf16 out, basis rows in registers)
            cb = pack_ops.dequantize_rows_int8(packed.coeff, packed.coeff_scale) if packed.coeff_quantized else packed.coeff.to(torch.bfloat16).contiguous()
            rows = cb.shape[0]
            out = stacr_ops.rebuild_input(cb, packed.basis.float().contiguous(), None, rows, hidden).clone().reshape(packed.original_shape)
        else:
            coeff = self._dequantize_coefficients(packed.coeff, packed.coeff_scale, packed.original_dtype) if packed.coeff_quantized else packed.coeff
            out = (coeff @ packed.basis.to(coeff.dtype).t()).reshape(packed.original_shape).to(packed.original_dtype)
        if not torch.isfinite(out).all():
            self.fallbacks["recon_nonfinite"] = self.fallbacks.get("recon_nonfinite", 0) + 1
            out = torch.nan_to_num(out)
        return out

    def stats(self) -> Dict[str, Any]:
        raw, stored = int(self._raw_bytes), int(self._stored_bytes)
        return {"site_id": self.spec.site_id, "packs": self.pack_count, "unpacks": self.unpack_count, "steps": self.step_count,
                "basis_refreshes": self.basis_refresh_count, "refresh_reasons": dict(self.refresh_reasons), "raw_bytes": raw,
                "stored_bytes": stored, "ratio": raw / stored if stored else None, "last_residual_energy": float(self._last_energy),
                "fallbacks": dict(self.fallbacks), "first_nonfinite": self.first_nonfinite}


class CheckpointSiteRegistry:
    def __init__(self):
        self.clear()

    def clear(self) -> None:
        self._by_module: Dict[int, STACRCheckpointSpec] = {}
        self._codecs: Dict[str, CheckpointBoundaryCodec] = {}

    def register(self, module: nn.Module, spec: STACRCheckpointSpec) -> None:
        self._by_module[id(module)] = spec
        codec = CheckpointBoundaryCodec(spec)
        self._codecs[spec.site_id] = codec
        module.add_module("_c1_codec", codec)  # so the codec's buffers travel with the model's state_dict

    def get(self, module: Optional[nn.Module]) -> Optional[STACRCheckpointSpec]:
        return None if module is None else self._by_module.get(id(module))

    def codec_for(self, site_id: str) -> Optional[CheckpointBoundaryCodec]:
        return self._codecs.get(site_id)

    def specs(self) -> Iterable[STACRCheckpointSpec]:
        return list(self._by_module.values())

    def items(self) -> Dict[str, CheckpointBoundaryCodec]:
        return dict(self._codecs)

    def __len__(self) -> int:
        return len(self._codecs)


_REGISTRY = CheckpointSiteRegistry()
_ACTIVE: Optional["STACRCheckpointRuntime"] = None


def get_global_checkpoint_site_registry() -> CheckpointSiteRegistry:
    return _REGISTRY


class STACRCheckpointRuntime:
    def __init__(self, registry: Optional[CheckpointSiteRegistry] = None):
        self.registry = registry or _REGISTRY
        self._active = False

    def is_active(self) -> bool:
        return self._active

    def activate(self) -> None:
        global _ACTIVE
        self._active, _ACTIVE = True, self

    def deactivate(self, *, clear_registry: bool = False) -> None:
        global _ACTIVE
        self._active = False
        if _ACTIVE is self:
            _ACTIVE = None
        if clear_registry:
            self.registry.clear()

    def resolve_site(self, function: Any) -> Optional[CheckpointBoundaryCodec]:
        module = getattr(function, "__self__", None)
        if module is None:
            module = getattr(getattr(function, "__wrapped__", None), "__self__", None)
        spec = self.registry.get(module)
        return self.registry.codec_for(spec.site_id) if spec else None

    def stats(self) -> Dict[str, Any]:
        per = {k: c.stats() for k, c in self.registry.items().items()}
        raw = sum(s["raw_bytes"] for s in per.values())
        stored = sum(s["stored_bytes"] for s in per.values())
        return {"sites": per, "raw_bytes": raw, "stored_bytes": stored, "ratio": raw / stored if stored else None}


def get_active_c1_runtime() -> Optional[STACRCheckpointRuntime]:
    return _ACTIVE if (_ACTIVE is not None and _ACTIVE.is_active()) else None


def clear_active_c1_runtime(*, clear_registry: bool = False) -> None:
    if _ACTIVE is not None:
        _ACTIVE.deactivate(clear_registry=clear_registry)


class _STACRCheckpointFunction(torch.autograd.Function):
    """Checkpoint whose boundary tensor (``args[target]``) is stored compressed."""

    @staticmethod
    def forward(ctx, run, codec, target, n_tensor, training, *flat):
        ctx.run, ctx.codec, ctx.target = run, codec, target
        tensors = list(flat[:n_tensor])
        ctx.record = codec.pack_tensor(tensors[target], training=training)
        ctx.others = [None if i == target else t for i, t in enumerate(tensors)]
        ctx.save_for_backward(*[t for i, t in enumerate(tensors) if i != target])
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if tensors[target].is_cuda else None
        ctx.autocast = (torch.is_autocast_enabled(tensors[target].device.type), torch.get_autocast_dtype(tensors[target].device.type))
        ctx.device_type = tensors[target].device.type
        ctx.records = []
        guard = get_global_recomputation_guard()
        with torch.no_grad(), guard.forward_context(ctx.records):
            out = run(*tensors)
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = iter(ctx.saved_tensors)
        tensors = []
        for i, slot in enumerate(ctx.others):
            if i == ctx.target:
                tensors.append(ctx.codec.unpack_record(ctx.record).detach().requires_grad_(True))
            else:
                t = next(saved)
                tensors.append(t.detach().requires_grad_(t.requires_grad) if t.is_floating_point() else t)
        guard = get_global_recomputation_guard()
        devices = [torch.cuda.current_device()] if ctx.cuda_rng is not None else []
        with torch.random.fork_rng(devices=devices):
            torch.set_rng_state(ctx.cpu_rng)
            if ctx.cuda_rng is not None:
                torch.cuda.set_rng_state(ctx.cuda_rng)
            with torch.enable_grad(), guard.recomputation_context(ctx.records), \
                    torch.autocast(ctx.device_type, dtype=ctx.autocast[1], enabled=ctx.autocast[0]):
                out = ctx.run(*tensors)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if isinstance(o, torch.Tensor) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        in_grads = [t.grad if isinstance(t, torch.Tensor) and t.requires_grad else None for t in tensors]
        return (None, None, None, None, None, *in_grads)


def stacr_checkpoint(function, *args, codec: CheckpointBoundaryCodec, target_arg_index: int = 0, training: bool = True, **kwargs):
    """Run ``function(*args, **kwargs)`` as a checkpoint whose ``args[target_arg_index]`` is kept compressed."""
    tensor_pos = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor)]
    if target_arg_index not in tensor_pos:
        raise ValueError("the boundary argument must be a tensor")

    def run(*tensors):
        full = list(args)
        for pos, t in zip(tensor_pos, tensors):
            full[pos] = t
        return function(*full, **kwargs)

    tensors = [args[i] for i in tensor_pos]
    return _STACRCheckpointFunction.apply(run, codec, tensor_pos.index(target_arg_index), len(tensors), training, *tensors)


def make_c1_saved_tensor_hooks(codec: CheckpointBoundaryCodec, *, training: bool = True):
    """Saved-tensor hooks that compress only tensors shaped like the site's boundary (hidden size match)."""

    def pack(t: torch.Tensor):
        if t.requires_grad and t.is_leaf:
            return t
        return codec.pack_tensor(t, training=training) if (t.dim() >= 2 and t.shape[-1] == codec.spec.hidden_size) else t

    def unpack(obj):
        return codec.unpack_record(obj) if isinstance(obj, CompressedBoundaryRecord) else obj

    return torch.autograd.graph.saved_tensors_hooks(pack, unpack)


_SITE_PATHS = (("transformer.h", "gpt2"), ("gpt_neox.layers", "neox"), ("model.layers", "llama"), ("bert.encoder.layer", "bert"),
               ("roberta.encoder.layer", "bert"))


def discover_checkpoint_sites(model: nn.Module) -> List[CheckpointSiteCandidate]:
    """Transformer blocks of GPT-2 / NeoX / LLaMA-style / BERT-style models, with their hidden size."""
    for path, family in _SITE_PATHS:
        try:
            stack = model.get_submodule(path)
        except AttributeError:
            continue
        cfg = getattr(model, "config", None)
        hidden = int(getattr(cfg, "hidden_size", getattr(cfg, "n_embd", 0)) or 0)
        if not hidden:
            first = next((m for m in stack[0].modules() if isinstance(m, nn.LayerNorm)), None)
            hidden = int(first.normalized_shape[0]) if first is not None else 0
        return [CheckpointSiteCandidate(f"{path}.{i}", blk, family, hidden) for i, blk in enumerate(stack)]
    return []


def enable_c1_checkpointing_for_model(model: nn.Module, config: STACRCheckpointConfig, *, amp_mode: str = "none",
                                      indices: Optional[Iterable[int]] = None) -> STACRCheckpointRuntime:
    """Wrap the selected blocks so their forward runs through :func:`stacr_checkpoint`.  Rejects parallel wrappers."""
    kind = type(model).__name__
    if kind in ("DataParallel", "DistributedDataParallel") or any(type(m).__name__ in ("TPGPT2MLP", "TPGPT2Attention") for m in model.modules()):
        raise ValueError("C1 checkpoint-boundary compression does not support tensor- or data-parallel wrapped models")
    sites = discover_checkpoint_sites(model)
    if not sites:
        raise ValueError("No checkpoint sites found for this architecture")
    device = next(model.parameters()).device
    registry = get_global_checkpoint_site_registry()
    registry.clear()
    runtime = STACRCheckpointRuntime(registry)
    chosen = set(range(len(sites))) if indices is None else set(indices)
    for i, site in enumerate(sites):
        if i not in chosen:
            continue
        rank = int(config.rank or _default_ckpt_rank(site.model_family, site.hidden_size))
        spec = STACRCheckpointSpec(
            site_id=site.name, module_type=type(site.module).__name__, model_family=site.model_family, hidden_size=site.hidden_size,
            rank=min(rank, site.hidden_size), residual_mode=config.residual_mode, residual_budget=config.residual_budget,
            basis_dtype=_resolve_ckpt_basis_dtype(config.basis_dtype, amp_mode, device), quantize_coefficients=config.quantize_coefficients,
            quantize_bits=config.quantize_bits, quantize_residuals=config.quantize_residuals, residual_quantize_bits=config.residual_quantize_bits,
            warmup_steps=config.warmup_steps, refresh_trigger=config.refresh_trigger, refresh_period=config.refresh_period,
            refresh_energy_threshold=_resolve_ckpt_refresh_energy_threshold(config.refresh_energy_threshold_mode, config.refresh_energy_threshold, rank, site.hidden_size),
            min_numel=config.min_numel,
        )
        registry.register(site.module, spec)
        codec = registry.codec_for(spec.site_id).to(device)
        inner = site.module.forward

        def forward(*args, __inner=inner, __codec=codec, __mod=site.module, **kwargs):
            if not (torch.is_grad_enabled() and __mod.training and isinstance(args[0], torch.Tensor) and args[0].requires_grad):
                return __inner(*args, **kwargs)
            return stacr_checkpoint(__inner, *args, codec=__codec, target_arg_index=0, training=True, **kwargs)

        site.module._c1_inner_forward = inner
        site.module.forward = forward
    runtime.activate()
    return runtime


# ------------------------------------------------------------------------------ registration from a run configuration
@dataclass
class ResolvedCheckpointSite:
    """A registered site at call time: the block, its spec and codec, and the boundary tensor among the call's arguments."""

    module: nn.Module
    spec: STACRCheckpointSpec
    codec: CheckpointBoundaryCodec
    target_tensor: Optional[torch.Tensor]
    target_arg_index: int = 0


def build_stacr_checkpoint_config(config: Any) -> STACRCheckpointConfig:
    """Collect a run configuration's ``stacr_ckpt_*`` attributes (and ``stacr_compress_checkpoint``) into a codec configuration.

    Parity: stacr/protocols/checkpointing.py:1186-1210.  Attributes the run configuration lacks keep the defaults.
    """
    defaults = STACRCheckpointConfig()
    picked = {}
    for f in dataclasses.fields(STACRCheckpointConfig):
        if f.name == "enabled":
            picked[f.name] = bool(getattr(config, "stacr_compress_checkpoint", False))
        else:
            value = getattr(config, f"stacr_ckpt_{f.name}", getattr(defaults, f.name))
            kind = type(getattr(defaults, f.name))
            picked[f.name] = value if value is None or kind is type(None) else kind(value)
    return STACRCheckpointConfig(**picked)


def _spec_for(site: CheckpointSiteCandidate, cfg: STACRCheckpointConfig, amp_mode: str, device: torch.device) -> STACRCheckpointSpec:
    rank = min(int(cfg.rank or _default_ckpt_rank(site.model_family, site.hidden_size)), site.hidden_size)
    return STACRCheckpointSpec(
        site_id=site.name, module_type=type(site.module).__name__, model_family=site.model_family, hidden_size=site.hidden_size, rank=rank,
        residual_mode=cfg.residual_mode, residual_budget=cfg.residual_budget, basis_dtype=_resolve_ckpt_basis_dtype(cfg.basis_dtype, amp_mode, device),
        quantize_coefficients=cfg.quantize_coefficients, quantize_bits=cfg.quantize_bits, quantize_residuals=cfg.quantize_residuals,
        residual_quantize_bits=cfg.residual_quantize_bits, warmup_steps=cfg.warmup_steps, refresh_trigger=cfg.refresh_trigger,
        refresh_period=cfg.refresh_period,
        refresh_energy_threshold=_resolve_ckpt_refresh_energy_threshold(cfg.refresh_energy_threshold_mode, cfg.refresh_energy_threshold, rank, site.hidden_size),
        min_numel=cfg.min_numel)


def collect_c1_site_candidates(model: nn.Module, config: Any) -> List[Tuple[CheckpointSiteCandidate, STACRCheckpointSpec]]:
    """Every transformer block that can carry a boundary codec, paired with the spec the run configuration gives it.

    Parity: stacr/protocols/checkpointing.py:1213-1296.  Raises when the architecture has no recognised block stack.
    """
    cfg = build_stacr_checkpoint_config(config)
    sites = discover_checkpoint_sites(model)
    if not sites:
        raise ValueError("checkpoint-boundary compression found no transformer blocks in this model")
    amp_mode = str(getattr(getattr(config, "baseline_cfg", None), "amp", "none") or "none")
    device = next(model.parameters()).device
    return [(site, _spec_for(site, cfg, amp_mode, device)) for site in sites]


def register_c1_sites(model: nn.Module, config: Any, *, runtime: Optional[STACRCheckpointRuntime] = None) -> STACRCheckpointRuntime:
    """Register a codec on each candidate block (after the byte planner's veto when it is set to ``enforce``).

    The blocks' forwards are left alone: a caller that checkpoints ``block.forward`` itself asks
    ``runtime.resolve_site(function)`` for the codec.  Parity: stacr/protocols/checkpointing.py:1299-1345.
    """
    runtime = runtime or STACRCheckpointRuntime()
    runtime.registry.clear()
    cfg = build_stacr_checkpoint_config(config)
    pairs = collect_c1_site_candidates(model, config)
    runtime.site_count_total = len(pairs)
    runtime.planner_mode, runtime.planner_summary, runtime.planner_decisions = cfg.planner, None, None
    keep = {site.name for site, _ in pairs}
    if cfg.planner != "off":
        from .planner import plan_stacr_checkpoint_sites, summarize_checkpoint_site_decisions

        decisions = plan_stacr_checkpoint_sites(model, config, [s.name for s, _ in pairs], pairs[0][0].hidden_size)
        runtime.planner_decisions = [d.to_dict() if hasattr(d, "to_dict") else dataclasses.asdict(d) for d in decisions]
        runtime.planner_summary = summarize_checkpoint_site_decisions(decisions)
        if cfg.planner == "enforce":
            keep = {d.name for d in decisions if d.keep}
            if not keep:
                reasons: Dict[str, int] = {}
                for d in decisions:
                    reasons[d.reason] = reasons.get(d.reason, 0) + 1
                raise ValueError("the byte planner rejected every checkpoint site: " + ", ".join(f"{k}={v}" for k, v in sorted(reasons.items())))
    device = next(model.parameters()).device
    for site, spec in pairs:
        if site.name in keep:
            runtime.registry.register(site.module, spec)
            runtime.registry.codec_for(spec.site_id).to(device)
    return runtime
