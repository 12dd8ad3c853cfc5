"""Protocol runner: one named training run with a method, a set of memory baselines and (optionally) DDP or TP.

``ConvergenceConfig`` mirrors the field names of the reference's runner configuration (the subset that selects
behaviour; unknown fields are rejected), ``run_convergence_experiment(cfg, logger)`` executes the run and writes
``config.json`` / ``metrics.jsonl`` / ``profile.jsonl`` / ``final.json`` through the logger.
Parity: experiments/protocols/training.py:146-5017 of the reference project (DDP helpers :442-528, target selection
:796-847, replacement :885-1471, baselines :2047-2144, validation :2560-2607, gradient cosine :2610-2742, per-layer
fidelity :3040-3215, spectrum telemetry :3314-3481, epoch loop :3484-4029, run :4032-5017).
"""

from __future__ import annotations

import copy
import math
import os
import time
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
from torch import nn

import stacr_b200 as S
from stacr_b200.adaptive import STACRConfig as AdaptiveConfig, STACRLinear as AdaptiveLinear, get_basis_pool, set_stacr_runtime_state
from stacr_b200.models import build_model
from stacr_b200.parallel import GradSync, broadcast_parameters
from stacr_b200.protocols.baselines.amp import AMPManager
from stacr_b200.protocols.baselines.checkpointing import apply_checkpointing
from stacr_b200.protocols.baselines.offload import OffloadManager
from stacr_b200.protocols.config.training import BaselineConfig
from stacr_b200.protocols.layers import CompressedLinear
from stacr_b200.protocols.planner import plan_stacr_layers, summarize_layer_decisions
from stacr_b200.protocols.prac import PRACConfig, replace_linear_with_prac, set_prac_global_step
from stacr_b200.protocols.profiling import PhaseProfiler
from stacr_b200.protocols.tensor_parallel import sync_replicated_grads
from stacr_b200.protocols.tp_gpt2 import TPActivationProfiler, apply_tensor_parallel_gpt2, disable_tp_dropout, get_tp_stacr_targets
from stacr_b200.protocols.utils import set_all_seeds

METHODS = ("baseline", "stacr", "stac", "svd", "tt", "tucker", "prac")


@dataclass
class ConvergenceConfig:
    """Every switch of a protocol run.  Field names follow the reference runner one for one so that published
    profile files load unchanged; ``train_examples``, ``eval_examples``, ``warmup_ratio``, ``model_overrides``,
    ``stacr_engine`` and ``stacr_surface`` exist only here."""

    experiment: str = "convergence_training"
    task: str = "synthetic_lm"           # synthetic_lm | wikitext103 | openwebtext | sst2 | ogbn-arxiv
    model: Optional[str] = "gpt2-medium"
    method: str = "baseline"
    method_label: Optional[str] = None
    run_tag: Optional[str] = "run"
    rank: int = 8
    reshape_shape: Optional[List[int]] = None
    factor_quantization_bits: Optional[int] = None
    factor_native_backward: bool = True
    use_lowrank_svd: bool = False
    tact_v3_config_path: Optional[str] = None
    tact_v3_target_ratio: int = 30
    baseline: Optional[str] = None
    baseline_cfg: Any = None
    epochs: int = 1
    batch_size: int = 8
    lr: float = 5e-5
    weight_decay: float = 0.0005
    momentum: float = 0.9
    max_length: int = 1024
    padding_mode: str = "dynamic"
    seed: int = 42
    deterministic: bool = True
    measure_memory: bool = True
    log_memory_both: bool = True
    monitor_grad_fidelity: bool = False
    grad_fidelity_interval: int = 100
    monitor_per_layer_grad_fidelity: bool = False
    per_layer_grad_fidelity_interval: int = 120
    monitor_svd_per_layer_grad_fidelity: bool = False
    svd_per_layer_grad_fidelity_interval: int = 240
    svd_per_layer_rank: Optional[int] = None
    svd_per_layer_oversampling: int = 16
    svd_per_layer_niter: int = 2
    monitor_reconstruction: bool = False
    reconstruction_interval: int = 240
    monitor_c1_drift: bool = True
    monitor_activation_spectrum: bool = False
    activation_spectrum_interval: int = 120
    activation_spectrum_rank: int = 8
    activation_spectrum_oversampling: int = 16
    activation_spectrum_niter: int = 2
    device: str = "auto"
    num_workers: int = 4
    use_data_parallel: bool = False
    use_ddp: bool = False
    use_tensor_parallel: bool = False
    use_8bit_optimizer: bool = False
    tp_scope: str = "full"
    tp_stacr_scope: str = "row_only"
    tp_profile_activations: bool = False
    max_steps: Optional[int] = 100
    train_examples: int = 512
    eval_examples: int = 32
    grad_clip: float = 0.0
    warmup_ratio: float = 0.1
    save_final_model: bool = False
    save_every_n_steps: Optional[int] = None
    debug_step_metrics_every: int = 0
    phase_profile_full_run: bool = False
    saved_tensors_compress_min_bytes: int = 100000
    saved_tensors_compress_dims: int = 4
    quiet: bool = True
    is_canonical_run: bool = False
    model_overrides: Dict[str, Any] = field(default_factory=dict)
    # ---- compression (adaptive engine); ``stacr_<x>`` feeds the engine option ``<x>`` unless _ENGINE_ALIASES renames it
    stacr_engine: str = "adaptive"
    stacr_surface: str = "mlp"
    stacr_residual_mode: str = "block_sparse"
    stacr_residual_budget: float = 0.005
    stacr_residual_threshold: float = 0.1
    stacr_update_trigger: str = "hybrid"
    stacr_update_interval: int = 100
    stacr_energy_threshold: float = 0.05
    stacr_streaming_algorithm: str = "oja"
    stacr_oja_learning_rate: float = 0.01
    stacr_warmup_steps: int = 0
    stacr_freeze_basis_after_warmup: bool = True
    stacr_quantize_coefficients: bool = True
    stacr_quantize_bits: int = 8
    stacr_quantize_residuals: bool = True
    stacr_residual_quantize_bits: int = 4
    stacr_randomized_svd_threshold: int = 1024
    stacr_randomized_svd_oversampling: int = 4
    stacr_randomized_svd_niter: int = 2
    stacr_adaptive_oja_lr: bool = False
    stacr_adaptive_oja_scale: float = 5.0
    stacr_adaptive_oja_max_lr: float = 0.1
    stacr_basis_dtype: str = "auto"
    stacr_backward_mode: str = "sparse"
    stacr_residual_block_size: int = 16
    stacr_cpu_offload: bool = False
    stacr_use_mgs: bool = False
    stacr_lazy_update: bool = True
    stacr_lazy_update_threshold: float = 0.01
    stacr_use_fused_kernel: bool = False
    stacr_rank_mode: str = "fixed"
    stacr_rank_variance_threshold: float = 0.95
    stacr_rank_min: int = 4
    stacr_rank_max: int = 64
    stacr_rank_adjust_interval: int = 100
    stacr_rank_sensitivity_low: float = 0.03
    stacr_rank_sensitivity_high: float = 0.1
    stacr_rank_step_fraction: float = 0.125
    stacr_streaming_topk: bool = False
    stacr_streaming_topk_sample_ratio: float = 0.1
    stacr_chunk_size: int = 512
    stacr_index_compression: str = "none"
    stacr_skip_residual: bool = False
    stacr_skip_residual_threshold: float = 0.05
    stacr_buffer_reuse: bool = False
    stacr_min_features: int = 256
    stacr_small_layer_rank_scale: float = 1.0
    stacr_small_layer_residual_scale: float = 1.0
    stacr_decoder_target_mode: str = "all"     # all | mlp_only | attention_only
    stacr_use_planner: bool = False
    stacr_planner_enforce: bool = False
    stacr_planner: str = "none"                # none | bytes (same as stacr_use_planner + stacr_planner_enforce)
    stacr_force_compress_layers: Optional[str] = None
    stacr_adaptive_layer_rank: str = "none"
    stacr_per_layer_rank_schedule: Optional[str] = None   # "c_fc=4,c_proj=12": rank by leaf-name substring
    stacr_residual_schedule: str = "none"
    stacr_residual_start: float = 0.05
    stacr_residual_end: float = 0.001
    stacr_post_warmup_mode: str = "full"
    stacr_post_warmup_residual_mode: Optional[str] = None  # alias of stacr_post_warmup_mode; wins when set
    stacr_residual_warmup_steps: int = 0
    stacr_post_warmup_threshold: float = 0.1
    stacr_refresh_trigger: str = "off"
    stacr_refresh_period: int = 1000
    stacr_refresh_energy_threshold: float = 0.1
    stacr_cache_basis_per_optimizer_step: bool = False
    stacr_oja_update_per_optimizer_step: bool = False
    stacr_enable_low_rank_only_fast_path: bool = True
    stacr_use_random_qr_init: bool = False
    stacr_min_adaptation_steps: int = 50
    stacr_allow_unadapted_random_qr: bool = False
    # ---- attention surface
    stacr_attention: bool = False
    stacr_attention_rank: Optional[int] = None
    stacr_attention_residual_mode: Optional[str] = None
    stacr_basis_sharing: str = "none"
    stacr_joint_qk: bool = False
    stacr_gpt2_split_c_attn: bool = False
    # ---- checkpoint-boundary compression
    stacr_compress_checkpoint: bool = False
    stacr_ckpt_target: str = "decoder_block_input"
    stacr_ckpt_rank: Optional[int] = None
    stacr_ckpt_warmup_steps: int = 500
    stacr_ckpt_residual_mode: str = "none"
    stacr_ckpt_residual_budget: float = 0.005
    stacr_ckpt_refresh_trigger: str = "residual_energy"
    stacr_ckpt_refresh_period: int = 200
    stacr_ckpt_refresh_energy_threshold_mode: str = "auto"
    stacr_ckpt_refresh_energy_threshold: float = 0.15
    stacr_ckpt_min_numel: int = 1 << 20
    stacr_ckpt_basis_dtype: str = "auto"
    stacr_ckpt_quantize_coefficients: bool = False
    stacr_ckpt_quantize_bits: int = 8
    stacr_ckpt_quantize_residuals: bool = True
    stacr_ckpt_residual_quantize_bits: int = 4
    stacr_ckpt_allow_inner_stacr: bool = False
    stacr_ckpt_planner: str = "heuristic"
    # ---- PRAC comparator
    prac_update_proj_gap: int = 50
    prac_seed_base: int = 42
    prac_proj_dtype: str = "auto"
    # ---- graph protocol (task ogbn-arxiv; read by experiments.protocols.graph)
    use_neighbor_sampling: bool = False
    num_neighbors: str = "30,30"
    use_random_node_loader: bool = False
    num_parts: int = 40
    use_stacr_graph: bool = False
    stacr_graph_tt_rank: int = 8
    stacr_graph_max_rank: int = 16
    stacr_graph_sparse_residual: bool = False
    stacr_graph_residual_budget: float = 0.1
    stacr_graph_residual_per_node: bool = False
    stacr_graph_chunk_size: int = 64
    stacr_graph_edge_eval_chunk_size: int = 100000
    stacr_graph_use_phantom: bool = False
    stacr_graph_phantom_samples: int = 5000
    stacr_graph_phantom_budget_frac: float = 0.2
    stacr_graph_phantom_seed: Optional[int] = None
    stacr_graph_use_hybrid: bool = False
    stacr_graph_hybrid_global_frac: float = 0.8
    stacr_graph_share_tt: bool = True
    stacr_graph_random_residual: bool = False
    stacr_graph_random_seed: int = 42
    stacr_graph_node_reorder: str = "none"
    # ---- convolutional comparators: accepted so that old profile files load; no convolutional model ships, so any
    # value other than the default is refused in __post_init__
    conv_compression_mode: str = "none"
    conv_compression_layers: str = "all"
    conv_skip_3x3: bool = True
    conv_min_channels: int = 64
    tucker_ranks: Optional[List[int]] = None
    conv_v2: bool = False
    conv_checkpoint: bool = False
    conv_block_checkpoint: bool = False
    conv_stage_checkpoint: bool = False
    conv_saved_hooks: bool = False
    conv_hooks_mode: str = "channel"

    def __post_init__(self):
        if os.environ.get("STACR_QUIET") == "1":
            self.quiet = True
        if self.method_label is None:
            self.method_label = self.method
        if self.method not in METHODS:
            raise ValueError(f"Unknown method {self.method!r}; choose from {METHODS}")
        if self.use_ddp and self.use_tensor_parallel:
            raise ValueError("Select DDP or tensor parallelism")
        if self.padding_mode not in ("dynamic", "max_length"):
            raise ValueError(f"padding_mode must be 'dynamic' or 'max_length', got {self.padding_mode}")
        if self.stacr_decoder_target_mode not in ("all", "mlp_only", "attention_only"):
            raise ValueError(f"Unknown stacr_decoder_target_mode {self.stacr_decoder_target_mode!r}")
        if self.conv_compression_mode != "none" or any((self.conv_v2, self.conv_checkpoint, self.conv_block_checkpoint, self.conv_stage_checkpoint, self.conv_saved_hooks)):
            raise ValueError("convolutional compression options need a convolutional model; none is available here")
        if isinstance(self.baseline_cfg, dict):
            self.baseline_cfg = BaselineConfig.from_mapping(self.baseline_cfg)
        elif self.baseline_cfg is None:
            self.baseline_cfg = BaselineConfig.from_legacy(self.baseline) if self.baseline not in (None, "none", "baseline") else BaselineConfig()
        if self.use_8bit_optimizer:
            self.baseline_cfg.optimizer_8bit = True
        if self.stacr_post_warmup_residual_mode is None:
            self.stacr_post_warmup_residual_mode = self.stacr_post_warmup_mode
        else:
            self.stacr_post_warmup_mode = self.stacr_post_warmup_residual_mode
        if self.stacr_use_planner and self.stacr_planner_enforce:
            self.stacr_planner = "bytes"
        if self.max_steps is None:
            self.max_steps = 1 << 62  # bounded by epochs * batches

    @classmethod
    def from_raw(cls, raw: Dict[str, Any]) -> "ConvergenceConfig":
        known = {f.name for f in fields(cls)}
        stray = sorted(set(raw) - known)
        if stray:
            raise ValueError(f"Unknown protocol fields: {stray}")
        return cls(**raw)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


# protocol field (without the ``stacr_`` prefix) -> engine option, where the names differ
_ENGINE_ALIASES = {
    "lazy_update": "lazy_update_enabled", "skip_residual": "skip_residual_enabled", "skip_residual_threshold": "skip_residual_energy_threshold",
    "post_warmup_mode": "post_warmup_residual_mode", "post_warmup_threshold": "post_warmup_residual_threshold",
}
# ``stacr_*`` fields that steer the runner, not the engine
_RUNNER_ONLY = {"engine", "surface", "min_features", "small_layer_rank_scale", "small_layer_residual_scale", "decoder_target_mode", "use_planner",
                "planner_enforce", "planner", "force_compress_layers", "per_layer_rank_schedule", "attention", "attention_rank",
                "attention_residual_mode", "gpt2_split_c_attn", "compress_checkpoint", "post_warmup_residual_mode"}


def parse_rank_schedule(text: Optional[str]) -> Dict[str, int]:
    """``"c_fc=4,c_proj=12"`` -> ``{"c_fc": 4, "c_proj": 12}``; a layer takes the rank of the first key its name contains."""
    out: Dict[str, int] = {}
    for item in (text or "").split(","):
        item = item.strip()
        if not item:
            continue
        key, sep, value = item.partition("=")
        if not sep or not key.strip() or int(value) < 1:
            raise ValueError(f"Bad rank schedule entry {item!r}; expected name=rank")
        out[key.strip()] = int(value)
    return out


# ------------------------------------------------------------------------------ distributed helpers
def init_ddp() -> tuple[int, int, int]:
    from stacr_b200.parallel import init_distributed

    return init_distributed()


def make_distributed_loader(batches: List[dict], rank: int, world: int) -> List[dict]:
    """Strided split: rank r takes batches r, r+world, ..."""
    return batches[rank::world] if world > 1 else batches


def _ddp_reduce_train_metrics(loss_sum: float, tokens: int, steps: int, peak: float, device) -> dict:
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return {"loss_sum": loss_sum, "tokens": tokens, "steps": steps, "peak_bytes": peak}
    sums = torch.tensor([loss_sum, tokens, steps], dtype=torch.float64, device=device)
    dist.all_reduce(sums)
    mx = torch.tensor([peak], dtype=torch.float32, device=device)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    return {"loss_sum": float(sums[0]), "tokens": int(sums[1]), "steps": int(sums[2]), "peak_bytes": float(mx)}


# ------------------------------------------------------------------------------ data
def build_batches(cfg: ConvergenceConfig, vocab: int, count: int, seed: int, device) -> List[dict]:
    gen = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(count):
        ids = torch.randint(0, vocab, (cfg.batch_size, cfg.max_length), generator=gen)
        batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids)}
        if cfg.task == "sst2":
            batch["labels"] = torch.bernoulli(torch.full((cfg.batch_size,), 0.5), generator=gen).long()
        else:
            batch["labels"] = ids.clone()
        out.append({k: v.to(device) for k, v in batch.items()})
    return out


# ------------------------------------------------------------------------------ targets and replacement
def select_targets(model: nn.Module, cfg: ConvergenceConfig) -> List[str]:
    if cfg.use_tensor_parallel:
        return get_tp_stacr_targets(model, cfg.tp_stacr_scope)
    surface = {"all": cfg.stacr_surface, "mlp_only": "mlp", "attention_only": "attention"}[cfg.stacr_decoder_target_mode]
    forced = [n.strip() for n in (cfg.stacr_force_compress_layers or "").split(",") if n.strip()]
    return S.select_target_names(model, surface=surface, min_features=cfg.stacr_min_features, extra_names=forced)


def _adaptive_config(cfg: ConvergenceConfig, **override) -> AdaptiveConfig:
    engine_fields = {f.name for f in fields(AdaptiveConfig)}
    opts: Dict[str, Any] = {"rank": cfg.rank}
    for f in fields(cfg):
        if not f.name.startswith("stacr_") or f.name.startswith(("stacr_ckpt_", "stacr_graph_")):
            continue
        short = f.name[len("stacr_"):]
        if short in _RUNNER_ONLY:
            continue
        target = _ENGINE_ALIASES.get(short, short)
        if target in engine_fields:
            opts[target] = getattr(cfg, f.name)
    opts["rank_max"] = max(int(opts.get("rank_max", 64)), int(opts.get("rank_min", 4)))
    if cfg.method == "stac":
        opts["residual_mode"] = "none"
    opts.update(override)
    return AdaptiveConfig(**opts)


def checkpoint_boundary_config(cfg: ConvergenceConfig):
    """The ``stacr_ckpt_*`` fields as a checkpoint-boundary codec configuration."""
    from stacr_b200.protocols.checkpointing import STACRCheckpointConfig

    names = {f.name for f in fields(STACRCheckpointConfig)}
    opts = {k[len("stacr_ckpt_"):]: v for k, v in cfg.to_dict().items() if k.startswith("stacr_ckpt_") and k[len("stacr_ckpt_"):] in names}
    return STACRCheckpointConfig(enabled=True, **opts)


def replace_linear_with_stacr(model: nn.Module, names: List[str], cfg: ConvergenceConfig) -> List[nn.Module]:
    """Wrap the named projections with the configured engine (adaptive by default, as the protocols do)."""
    if cfg.stacr_engine == "projection":
        return S.apply_stacr(model, surface="none", target_names=names, rank=cfg.rank, residual_budget=cfg.stacr_residual_budget,
                             turbo_after_step=None, allow_empty=True)
    base = _adaptive_config(cfg)
    schedule = parse_rank_schedule(cfg.stacr_per_layer_rank_schedule)
    layers = []
    for i, name in enumerate(names):
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        source = getattr(parent, leaf)
        conf = copy.deepcopy(base)
        feats = int(source.weight.shape[0] if type(source).__name__ == "Conv1D" else source.weight.shape[1])
        for key, value in schedule.items():
            if key in name:
                conf.rank = min(value, feats)
                break
        else:
            if feats < 1024 and cfg.stacr_small_layer_rank_scale != 1.0:
                conf.rank = max(1, min(feats, int(round(conf.rank * cfg.stacr_small_layer_rank_scale))))
        if feats < 1024 and cfg.stacr_small_layer_residual_scale != 1.0:
            conf.residual_budget = min(1.0, conf.residual_budget * cfg.stacr_small_layer_residual_scale)
        conf.rank_max = max(conf.rank_max, conf.rank)
        layer = AdaptiveLinear.from_linear(source, conf, layer_index=i, num_layers=len(names))
        layer.source_name = name
        setattr(parent, leaf, layer)
        layers.append(layer)
    return layers


def compress_attention_surface(model: nn.Module, cfg: ConvergenceConfig):
    """``stacr_attention``: wrap the Q/K/V projections too (own rank / residual mode when given)."""
    from stacr_b200.protocols.attention import apply_stacr_to_attention

    extra = {}
    if cfg.stacr_attention_rank is not None:
        extra["rank"] = int(cfg.stacr_attention_rank)
    if cfg.stacr_attention_residual_mode is not None:
        extra["residual_mode"] = cfg.stacr_attention_residual_mode
    conf = _adaptive_config(cfg, **extra)
    conf.rank_max = max(conf.rank_max, conf.rank)
    return apply_stacr_to_attention(model, conf, enable_gpt2_c_attn_split=cfg.stacr_gpt2_split_c_attn, mask_aware=cfg.padding_mode == "max_length",
                                    joint_qk=cfg.stacr_joint_qk)


def replace_linear_with_compressed(model: nn.Module, names: List[str], cfg: ConvergenceConfig) -> List[nn.Module]:
    """SVD / TT / Tucker comparators on the same targets."""
    out = []
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        lin = getattr(parent, leaf)
        if not isinstance(lin, nn.Linear):
            continue
        rows = cfg.batch_size * cfg.max_length
        conf: Dict[str, Any] = {"method": cfg.method, "rank": cfg.rank, "quantize_bits": cfg.factor_quantization_bits, "use_lowrank": cfg.use_lowrank_svd}
        if cfg.method in ("tt", "tucker"):
            shape = cfg.reshape_shape or _default_tensor_shape(rows, lin.in_features)
            conf["reshape_shape"] = tuple(shape)
            conf["ranks"] = [min(cfg.rank, d) for d in shape]
        wrapped = CompressedLinear.from_linear(lin, conf)
        setattr(parent, leaf, wrapped)
        out.append(wrapped)
    return out


def _default_tensor_shape(rows: int, feats: int):
    def two(n):
        a = int(math.isqrt(n))
        while a > 1 and n % a:
            a -= 1
        return [a, n // a]
    return two(rows) + two(feats)


# ------------------------------------------------------------------------------ baselines
def data_parallel_blockers(cfg: ConvergenceConfig, device) -> List[str]:
    """Why the legacy single-process ``nn.DataParallel`` arm cannot run this configuration (empty = it can).

    The arm replicates the module per forward and scatters the batch, so it is limited to plain SST-2 / WikiText runs without
    anything that keeps per-module state across the replicas (checkpoint wrappers, quantised-activation libraries, saved-tensor
    offload, boundary compression) and without gradient accumulation (experiments/protocols/training.py:2063-2100 of the reference).
    """
    b = cfg.baseline_cfg
    why = []
    if torch.device(device).type != "cuda":
        why.append("non-CUDA device")
    if (torch.cuda.device_count() if torch.cuda.is_available() else 0) < 2:
        why.append("fewer than 2 CUDA devices")
    if cfg.task not in ("sst2", "wikitext103"):
        why.append(f"task={cfg.task}")
    if b.checkpointing != "none":
        why.append("checkpointing")
    for key in ("actnn", "gact", "torchao"):
        if getattr(b, key, "none") != "none":
            why.append(key)
    if b.offload != "none":
        why.append("saved_tensors_offload")
    if cfg.stacr_compress_checkpoint or b.c1_checkpoint_compression:
        why.append("stacr_compress_checkpoint")
    if int(b.grad_accum_steps) > 1:
        why.append("grad_accum_steps > 1")
    return why


def apply_baseline(model: nn.Module, cfg: ConvergenceConfig, device) -> Dict[str, Any]:
    b = cfg.baseline_cfg
    state: Dict[str, Any] = {"amp": AMPManager(b.amp, str(device)), "offload": None, "checkpointed": 0}
    if cfg.use_data_parallel:
        blockers = data_parallel_blockers(cfg, device)
        if blockers:
            state["status"] = "skipped_incompatible"
            state["reason"] = "DataParallel is limited to simple SST-2/WikiText runs; incompatible with: " + ", ".join(blockers)
            return state
    if b.checkpointing != "none":
        state["checkpointed"] = apply_checkpointing(model, b.checkpointing)
    for key, module_name, fn_name in (("actnn", "actnn_adapter", "try_enable_actnn"), ("gact", "gact_adapter", "try_enable_gact")):
        level = getattr(b, key)
        if level != "none":
            import importlib

            adapter = importlib.import_module(f"stacr_b200.protocols.baselines.{module_name}")
            _, outcome = getattr(adapter, fn_name)(model, level)
            state[key] = outcome.to_dict() if hasattr(outcome, "to_dict") else str(outcome)
    if b.offload != "none":
        state["offload"] = OffloadManager(b.offload, b.offload_min_bytes)
    if b.c1_checkpoint_compression:
        from stacr_b200.protocols.checkpointing import STACRCheckpointConfig, enable_c1_checkpointing_for_model

        state["c1"] = enable_c1_checkpointing_for_model(model, STACRCheckpointConfig(enabled=True, warmup_steps=0, min_numel=0), amp_mode=b.amp)
    elif cfg.stacr_compress_checkpoint:
        from stacr_b200.protocols.checkpointing import enable_c1_checkpointing_for_model

        state["c1"] = enable_c1_checkpointing_for_model(model, checkpoint_boundary_config(cfg), amp_mode=b.amp)
    return state


def build_optimizer(model: nn.Module, cfg: ConvergenceConfig):
    params = [p for p in model.parameters() if p.requires_grad]
    galore = cfg.baseline_cfg.galore_options()
    if galore is not None:
        from stacr_b200.comparators.galore_adapter import create_galore_optimizer

        return create_galore_optimizer(model, lr=cfg.lr, weight_decay=cfg.weight_decay, **galore), f"GaLoreAdamW({cfg.baseline_cfg.galore})"
    if cfg.baseline_cfg.torchao not in ("none", "float8"):
        from stacr_b200.protocols.baselines.torchao_adapter import try_create_torchao_optimizer

        name = "adamw8bit" if cfg.baseline_cfg.torchao == "auto" else cfg.baseline_cfg.torchao
        made, result = try_create_torchao_optimizer(params, name, lr=cfg.lr, weight_decay=cfg.weight_decay)
        if made is not None:
            return made, f"torchao:{name}"
    if cfg.baseline_cfg.optimizer_8bit:
        from stacr_b200.optim import AdamW8bit

        return AdamW8bit(params, lr=cfg.lr, weight_decay=cfg.weight_decay), "AdamW8bit(in-tree)"
    if params[0].is_cuda:
        from stacr_b200.optim import AdamW

        return AdamW(params, lr=cfg.lr, weight_decay=cfg.weight_decay), "AdamW(in-tree)"
    return torch.optim.AdamW(params, lr=cfg.lr, weight_decay=cfg.weight_decay), "AdamW"


# ------------------------------------------------------------------------------ telemetry
@torch.no_grad()
def validate(model, batches, amp: AMPManager, task: str) -> Dict[str, float]:
    was = model.training
    model.eval()
    nll = n = correct = seen = 0
    for batch in batches:
        with amp.autocast():
            out = model(**batch)
        if task == "sst2":
            correct += int((out.logits.argmax(-1) == batch["labels"]).sum())
            seen += batch["labels"].numel()
        else:
            nll += float(out.loss)
            n += 1
    model.train(was)
    if task == "sst2":
        return {"val_accuracy": 100.0 * correct / max(1, seen)}
    mean = nll / max(1, n)
    return {"val_loss": mean, "val_ppl": math.exp(min(700.0, mean))}


def compute_grad_cosine(model, batch, amp: AMPManager) -> Optional[float]:
    """Cosine between the gradient through the actual (compressed) backward and the exact gradient on one batch."""
    from stacr_b200.diagnostics import compression_diagnostics

    params = [p for p in model.parameters() if p.requires_grad]
    stash = [None if p.grad is None else p.grad.clone() for p in params]

    def grads(compress: bool):
        model.zero_grad(set_to_none=True)
        flags = {m: m.training for m in model.modules()}
        try:
            if compress:
                with compression_diagnostics(model), amp.autocast():
                    model(**batch).loss.backward()
            else:
                model.eval()  # compressed layers take their exact path in eval mode
                with amp.autocast():
                    model(**batch).loss.backward()
        finally:
            for m, f in flags.items():
                m.training = f
        return torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).double() for p in params])

    try:
        exact, approx = grads(False), grads(True)
        value = float(S.cosine_similarity(exact, approx))
    except ValueError:
        value = None
    for p, g in zip(params, stash):
        p.grad = g
    return value


def compute_per_layer_grad_fidelity(model, batch, amp: AMPManager, layers) -> Dict[str, float]:
    """Per wrapped layer: cosine between exact and compressed weight gradients on one batch."""
    from stacr_b200.diagnostics import compression_diagnostics

    def weight_of(layer):
        if isinstance(layer, AdaptiveLinear):
            lin = layer.linear
            return getattr(lin, "source_weight", None) if hasattr(lin, "source_weight") else lin.weight
        if hasattr(layer, "weight"):
            return layer.weight
        return layer.linear.weight  # comparator wrappers keep the dense projection as ``linear``

    weights = {getattr(l, "source_name", str(i)): weight_of(l) for i, l in enumerate(layers)}
    stash = {k: (None if w.grad is None else w.grad.clone()) for k, w in weights.items()}
    out: Dict[str, float] = {}
    flags = {m: m.training for m in model.modules()}
    try:
        model.zero_grad(set_to_none=True)
        model.eval()
        with amp.autocast():
            model(**batch).loss.backward()
        exact = {k: w.grad.detach().clone() for k, w in weights.items() if w.grad is not None}
        for m, f in flags.items():
            m.training = f
        model.zero_grad(set_to_none=True)
        with compression_diagnostics(model), amp.autocast():
            model(**batch).loss.backward()
        for k, w in weights.items():
            if k in exact and w.grad is not None:
                out[k] = float(S.cosine_similarity(exact[k], w.grad))
    finally:
        for m, f in flags.items():
            m.training = f
        for k, w in weights.items():
            w.grad = stash[k]
    return out


def compute_activation_spectrum_telemetry(model, batch, amp: AMPManager, layers, rank: int = 8) -> Dict[str, dict]:
    """Energy captured by the top-``rank`` singular directions of each wrapped layer's input on one batch."""
    captured: Dict[str, torch.Tensor] = {}
    hooks = []
    for i, layer in enumerate(layers):
        name = getattr(layer, "source_name", str(i))
        hooks.append(layer.register_forward_pre_hook(lambda m, inp, _n=name: captured.__setitem__(_n, inp[0].detach())))
    was = model.training
    model.eval()
    with torch.no_grad(), amp.autocast():
        model(**batch)
    model.train(was)
    for h in hooks:
        h.remove()
    out = {}
    for name, x in captured.items():
        s = torch.linalg.svdvals(x.reshape(-1, x.shape[-1]).float()[:4096])
        e = s.square()
        out[name] = {"top_rank_energy": float(e[:rank].sum() / e.sum().clamp_min(1e-30)), "stable_rank": float(e.sum() / e[0].clamp_min(1e-30))}
    return out


# ------------------------------------------------------------------------------ the run
def run_convergence_experiment(cfg: ConvergenceConfig, logger) -> Dict[str, Any]:
    get_basis_pool().clear()
    set_all_seeds(cfg.seed, strict=False)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    cuda = torch.cuda.is_available() and cfg.device in ("auto", "cuda")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
    logger.write_config(cfg.to_dict())
    model_name = cfg.model or ("bert-base-uncased" if cfg.task == "sst2" else "gpt2-medium")
    model = build_model(model_name, **cfg.model_overrides).to(device).train()
    vocab = model.config.vocab_size
    tp_profiler = None
    if cfg.use_tensor_parallel:
        if world < 2 and not cfg.quiet:
            print("[TP] single rank: sharding degenerates to the unsharded model")
        apply_tensor_parallel_gpt2(model, rank, world, None, scope=cfg.tp_scope)
        disable_tp_dropout(model)
        if cfg.tp_profile_activations:
            tp_profiler = TPActivationProfiler(model)
    elif cfg.use_ddp:
        broadcast_parameters(model)
    layers: List[nn.Module] = []
    plan_summary = None
    attention_report = None
    if cfg.method in ("stacr", "stac"):
        names = select_targets(model, cfg)
        if cfg.stacr_planner == "bytes":
            decisions = plan_stacr_layers(model, cfg, names)
            plan_summary = summarize_layer_decisions(decisions)
            names = [d.name for d in decisions if d.keep]
        layers = replace_linear_with_stacr(model, names, cfg)
        if cfg.stacr_attention and cfg.stacr_engine == "adaptive":
            attention_report = compress_attention_surface(model, cfg)
            layers += [m for m in model.modules() if isinstance(m, AdaptiveLinear) and m not in layers]
    elif cfg.method in ("svd", "tt", "tucker"):
        layers = replace_linear_with_compressed(model, select_targets(model, cfg), cfg)
    elif cfg.method == "prac":
        layers = replace_linear_with_prac(model, select_targets(model, cfg), PRACConfig(rank=cfg.rank, update_proj_gap=cfg.prac_update_proj_gap, seed_base=cfg.prac_seed_base,
                                                                                    proj_dtype=None if cfg.prac_proj_dtype == "auto" else cfg.prac_proj_dtype, quiet=True))
    state = apply_baseline(model, cfg, device)
    if state.get("status") == "skipped_incompatible":
        final = {"status": "skipped_incompatible", "reason": state["reason"], "run_tag": cfg.run_tag, "method": cfg.method, "model": cfg.model, "steps": 0}
        logger.write_final(final)
        return final
    amp: AMPManager = state["amp"]
    optimizer, optimizer_name = build_optimizer(model, cfg)
    train_model_ref = model
    if cfg.use_data_parallel and cuda and torch.cuda.device_count() > 1:
        # the legacy single-process arm: replicas per forward, batch scattered over the visible GPUs, gradients summed on device 0
        train_model_ref = torch.nn.DataParallel(model)
    from .diagnostics import C1DriftTracker, reconstruction_report

    drift = C1DriftTracker() if (state.get("c1") is not None and cfg.monitor_c1_drift) else None
    sync = GradSync(model.parameters()) if (cfg.use_ddp and world > 1) else None
    profiler = PhaseProfiler(out_path=logger.profile_path, enabled=cfg.phase_profile_full_run and logger.profile_path is not None)
    for layer in layers:
        if isinstance(layer, AdaptiveLinear):
            layer.phase_profiler = profiler
    data_world = world if cfg.use_ddp else 1
    train = make_distributed_loader(build_batches(cfg, vocab, max(1, cfg.train_examples // cfg.batch_size), cfg.seed, device), rank if cfg.use_ddp else 0, data_world)
    val = build_batches(cfg, vocab, max(1, cfg.eval_examples // cfg.batch_size), cfg.seed + 1, device)
    accum = int(cfg.baseline_cfg.grad_accum_steps)
    total_steps = min(cfg.max_steps, max(1, cfg.epochs * len(train) // accum))
    warm = int(cfg.warmup_ratio * total_steps)
    if cuda:
        torch.cuda.reset_peak_memory_stats(device)
    step = 0
    loss_sum, tokens = 0.0, 0
    history: List[float] = []
    t0 = time.perf_counter()
    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) if cuda else None
    if ev:
        ev[0].record()
    status = "ok"
    try:
        while step < total_steps:
            batch = train[step % len(train)]
            lr_scale = min(1.0, (step + 1) / max(1, warm)) if step < warm else max(0.0, (total_steps - step) / max(1, total_steps - warm))
            for g in optimizer.param_groups:
                g["lr"] = cfg.lr * lr_scale
            S.set_step([l for l in layers if isinstance(l, S.STACRLinear)], step)
            if cfg.method == "prac":
                set_prac_global_step(model, step)
            with profiler.step(step):
                sync.zero_grad() if sync else optimizer.zero_grad(set_to_none=True)
                ctx = state["offload"].training_step() if state["offload"] else _null()
                with ctx:
                    value = 0.0
                    for micro in range(accum):
                        batch = train[(step * accum + micro) % len(train)]
                        set_stacr_runtime_state(model, step, micro, accum, total_steps)
                        with profiler.phase("forward"), amp.autocast():
                            loss = train_model_ref(**batch).loss
                            loss = (loss.mean() if loss.dim() else loss) / accum
                        value += float(loss.detach())
                        if not math.isfinite(value):
                            raise FloatingPointError(f"Nonfinite loss at step {step}")
                        with profiler.phase("backward"):
                            amp.backward(loss)
                with profiler.phase("optimizer"):
                    if sync:
                        sync.finish()
                    if cfg.use_tensor_parallel and world > 1:
                        sync_replicated_grads(model, None)
                    if cfg.grad_clip > 0:
                        amp.unscale_(optimizer)
                        torch.nn.utils.clip_grad_norm_(model.parameters(), cfg.grad_clip)
                    amp.step(optimizer)
            loss_sum += value
            tokens += int(batch["attention_mask"].sum())
            history.append(value)
            record = {"step": step, "train_loss": value, "lr": cfg.lr * lr_scale}
            if cfg.monitor_grad_fidelity and layers and step % cfg.grad_fidelity_interval == 0:
                record["grad_cosine"] = compute_grad_cosine(model, batch, amp)
            if cfg.monitor_per_layer_grad_fidelity and layers and step % cfg.per_layer_grad_fidelity_interval == 0:
                record["per_layer_grad_cosine"] = compute_per_layer_grad_fidelity(model, batch, amp, layers)
            if cfg.monitor_activation_spectrum and layers and step % cfg.activation_spectrum_interval == 0:
                record["activation_spectrum"] = compute_activation_spectrum_telemetry(model, batch, amp, layers, cfg.activation_spectrum_rank)
            if cfg.monitor_reconstruction and layers and step % cfg.reconstruction_interval == 0:
                def _fwd(batch=batch):
                    with torch.no_grad(), amp.autocast():
                        model(**batch)
                record["reconstruction"] = reconstruction_report(model, layers, _fwd, cfg.svd_per_layer_rank)["summary"]
            if drift is not None:
                record["c1_drift"] = drift.update(state["c1"].stats(), global_step=step, optimizer_step=step, loss_value=value)
                if cuda:
                    drift.note_memory("after_step", torch.cuda.memory_allocated(device))
            logger.log(record)
            step += 1
            if cfg.save_every_n_steps and step % cfg.save_every_n_steps == 0:
                if int(os.environ.get("LOCAL_RANK", "0")) == 0 and getattr(logger, "dir", None):
                    target = logger.dir / f"checkpoint_step_{step}"
                    target.mkdir(parents=True, exist_ok=True)
                    torch.save(model.state_dict(), target / "model.pt")
                if world > 1 and torch.distributed.is_initialized():
                    # the other ranks wait on the host while one rank writes: the device-side peer waits of the next
                    # step's collectives are bounded and must not be spent on a checkpoint
                    torch.distributed.barrier()
    except FloatingPointError as exc:
        status = f"error: {exc}"
    if ev:
        ev[1].record()
        torch.cuda.synchronize(device)
        elapsed = ev[0].elapsed_time(ev[1]) / 1e3
    else:
        elapsed = time.perf_counter() - t0
    peak = float(torch.cuda.max_memory_allocated(device)) if cuda else 0.0
    reduced = _ddp_reduce_train_metrics(loss_sum, tokens, step, peak, device)
    quality = validate(model, val, amp, cfg.task) if (rank == 0 or cfg.use_tensor_parallel) else {}
    flags: Dict[str, Any] = {}
    adaptive = [l for l in layers if isinstance(l, AdaptiveLinear)]
    if adaptive:
        flags = {
            "basis_updates": sum(l.layer_state["basis_updates"] for l in adaptive),
            "refresh_count_total": sum(l.layer_state["refresh_count_total"] for l in adaptive),
            "mean_residual_energy": sum(float(l.layer_state["last_residual_energy"]) for l in adaptive) / len(adaptive),
            "active_ranks": [int(l.layer_state["active_rank"]) for l in adaptive],
            "low_rank_only_steps": sum(l.layer_state["b1_route_step_count"] for l in adaptive),
        }
    final = {
        "status": status, "run_tag": cfg.run_tag, "method": cfg.method, "model": cfg.model, "world_size": world, "steps": step,
        "optimizer": optimizer_name, "train_loss_mean": reduced["loss_sum"] / max(1, reduced["steps"]), "train_loss_last": history[-1] if history else None,
        "train_loss_first": history[0] if history else None, "seconds": elapsed, "tokens_per_second": reduced["tokens"] / elapsed if elapsed > 0 else None,
        "peak_allocated_bytes": reduced["peak_bytes"], "n_wrapped_layers": len(layers), "baseline": cfg.baseline_cfg.get_description(),
        "stacr_flags": flags, "planner": plan_summary, "attention": attention_report.to_dict() if attention_report else None, "tp_activation_profile": tp_profiler.summary() if tp_profiler else None,
        "offload": state["offload"].get_stats() if state["offload"] else None, **quality,
        "c1_drift": drift.summary() if drift is not None else None, "data_parallel": bool(train_model_ref is not model),
    }
    if cfg.save_final_model and int(os.environ.get("LOCAL_RANK", "0")) == 0 and getattr(logger, "dir", None):
        (logger.dir / "checkpoint").mkdir(parents=True, exist_ok=True)
        torch.save(model.state_dict(), logger.dir / "checkpoint" / "model.pt")
    logger.write_final(final)
    if sync:
        sync.close()
    return final


class _null:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


from .training_helpers import *  # noqa: E402,F401,F403  (stand-alone pieces of the protocol, part of this module's API)
from .training_helpers import __all__ as _HELPER_NAMES  # noqa: E402
