"""Model surgery: choose linear projections by saved-activation surface and wrap them.

API parity with stacr/surgery.py:15-259 of the reference project: ``classify``,
``select_target_names``, ``apply_stacr`` (plan first, mutate last; shared modules wrapped once),
``set_step`` (both engines, with micro-batch position).
"""

from __future__ import annotations

import inspect
import re
from dataclasses import asdict, is_dataclass
from typing import Any, Iterable

from torch import nn

from .layers import STACRLinear

# Surfaces are decided by the *parent* block: GPT-2 calls both the MLP output and the attention
# output "c_proj", BERT calls both "dense".
MLP_PARENTS = ("mlp", "ffn", "feed_forward", "intermediate")
ATTENTION_PARENTS = ("attn", "attention", "self_attn", "self_attention", "crossattention")
MLP_LEAVES = (
    "c_fc", "c_proj", "dense", "dense_h_to_4h", "dense_4h_to_h", "gate_proj", "up_proj", "down_proj",
    "fc1", "fc2", "w1", "w2", "w3",
)
ATTENTION_LEAVES = (
    "c_attn", "c_proj", "dense", "q_proj", "k_proj", "v_proj", "o_proj", "out_proj", "query", "key", "value",
    "query_key_value",
)
# OPT hangs fc1/fc2 directly on the decoder layer (no mlp parent); these two leaf names never
# denote attention projections, so they may be classified by leaf alone.
UNAMBIGUOUS_MLP_LEAVES = ("fc1", "fc2")

_SURFACES = {"mlp": {"mlp"}, "attention": {"attention"}, "mlp+attention": {"mlp", "attention"}, "all": None, "none": set()}
_SELECTION_KEYS = frozenset(
    {"surface", "min_features", "extra_names", "target_names", "target_pattern", "exclude_names", "trainable_only", "allow_empty"}
)
_COMPAT_KEYS = frozenset({"min_numel", "post_warmup_mode"})  # accepted so the hook-path config dataclass can be passed


def _is_conv1d(module: nn.Module) -> bool:
    return type(module).__name__ == "Conv1D" and hasattr(module, "weight") and module.weight.dim() == 2


def _in_features(module: nn.Module) -> int | None:
    if isinstance(module, nn.Linear):
        return int(module.in_features)
    if _is_conv1d(module):
        return int(module.weight.shape[0])
    return None


def classify(name: str) -> str | None:
    """``'attention'``, ``'mlp'`` or ``None`` for a dotted module name."""
    *parents, leaf = name.split(".")
    above = set(parents)
    if above.intersection(ATTENTION_PARENTS):
        return "attention" if leaf in ATTENTION_LEAVES else None
    if above.intersection(MLP_PARENTS) or "output" in above:
        return "mlp" if leaf in MLP_LEAVES else None
    return "mlp" if leaf in UNAMBIGUOUS_MLP_LEAVES else None


def _as_set(values) -> set[str]:
    return {values} if isinstance(values, str) else set(values)


def select_target_names(
    model: nn.Module,
    *,
    surface: str = "mlp",
    min_features: int = 256,
    extra_names: Iterable[str] = (),
    target_names: Iterable[str] | None = None,
    target_pattern: str | None = None,
    exclude_names: Iterable[str] = (),
    trainable_only: bool = True,
) -> list[str]:
    """Names of the linear projections to compress.

    ``target_names`` / ``target_pattern`` restrict the candidates; ``extra_names`` add to a
    surface (``surface='none'`` plus extras gives a purely explicit list).  Explicitly named
    modules bypass ``min_features``.
    """
    if surface not in _SURFACES:
        raise ValueError(f"Unknown surface: {surface!r}")
    if isinstance(min_features, bool) or int(min_features) != min_features or min_features < 1:
        raise ValueError("min_features must be a positive integer")
    extras = _as_set(extra_names)
    only = None if target_names is None else _as_set(target_names)
    skip = _as_set(exclude_names)
    regex = re.compile(target_pattern) if target_pattern is not None else None
    named = dict(model.named_modules(remove_duplicate=False))
    explicit = extras | (only or set())
    unknown = explicit - named.keys()
    if unknown:
        raise ValueError(f"Unknown target module names: {sorted(unknown)}")
    not_linear = sorted(n for n in explicit if _in_features(named[n]) is None)
    if not_linear:
        raise ValueError(f"Targets are not supported linear projections: {not_linear}")
    wanted = _SURFACES[surface]
    chosen: list[str] = []
    for name, module in named.items():
        width = _in_features(module)
        if width is None or name in skip:
            continue
        if trainable_only and not module.weight.requires_grad:
            continue
        if only is not None and name not in only:
            continue
        if regex is not None and regex.search(name) is None:
            continue
        if width < int(min_features) and name not in explicit:
            continue
        forced = surface == "all" or name in explicit or only is not None or regex is not None
        if forced or (wanted and classify(name) in wanted):
            chosen.append(name)
    return chosen


def _layer_option_names() -> set[str]:
    return set(inspect.signature(STACRLinear.__init__).parameters) - {"self", "weight", "bias", "transposed"}


def apply_stacr(model: nn.Module, config: dict[str, Any] | None = None, **overrides: Any) -> list[STACRLinear]:
    """Wrap the selected projections of ``model`` in place and return the new layers.

    Defaults to Turbo-fast: at optimizer step 50 the basis freezes and residual storage stops
    (weights keep training).  ``turbo_after_step=None`` keeps full STAC-R; a config dataclass that
    carries an explicit ``None`` therefore selects full STAC-R.  Call ``set_step`` each step.
    """
    options: dict[str, Any] = asdict(config) if is_dataclass(config) else dict(config or {})
    options.update(overrides)
    options.setdefault("turbo_after_step", 50)
    layer_keys = _layer_option_names()
    stray = options.keys() - layer_keys - _SELECTION_KEYS - _COMPAT_KEYS
    if stray:
        raise ValueError(f"Unknown STAC-R options: {sorted(stray)}")
    if options.get("post_warmup_mode", "full") != "full":
        raise ValueError("Use turbo_after_step to switch the factor-native layer to Turbo")
    names = select_target_names(
        model,
        surface=str(options.get("surface", "mlp")),
        min_features=options.get("min_features", 256),
        extra_names=options.get("extra_names", ()),
        target_names=options.get("target_names"),
        target_pattern=options.get("target_pattern"),
        exclude_names=options.get("exclude_names", ()),
        trainable_only=options.get("trainable_only", True),
    )
    if "" in names:
        raise ValueError("For a standalone linear module use STACRLinear.from_linear(model, ...)")
    if not names and not options.get("allow_empty", False) and options.get("surface") != "none":
        raise ValueError(
            "No trainable linear projections matched. Select surface='all', supply "
            "target_names, lower min_features, or explicitly set allow_empty=True."
        )
    layer_kwargs = {k: options[k] for k in layer_keys if k in options}
    # Phase 1: build every wrapper (any invalid option raises here, model untouched).
    by_module: dict[int, STACRLinear] = {}
    edits: list[tuple[nn.Module, str, STACRLinear]] = []
    for name in names:
        parent_path, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_path) if parent_path else model
        original = getattr(parent, leaf)
        wrapper = by_module.get(id(original))
        if wrapper is None:
            wrapper = STACRLinear.from_linear(original, **layer_kwargs)
            wrapper.source_name = name
            by_module[id(original)] = wrapper
        edits.append((parent, leaf, wrapper))
    # Phase 2: rebind; aliases of a shared module all point at its single wrapper.
    ordered: list[STACRLinear] = []
    for parent, leaf, wrapper in edits:
        setattr(parent, leaf, wrapper)
        if not any(wrapper is w for w in ordered):
            ordered.append(wrapper)
    return ordered


def set_step(layers: Iterable[nn.Module] | nn.Module, step: int, *, microbatch_index: int = 0, accum_steps: int = 1) -> None:
    """Publish the optimizer step (and micro-batch position) to compressed layers of either engine."""
    from .adaptive import STACRLinear as AdaptiveLinear

    if isinstance(step, bool) or int(step) != step or step < 0:
        raise ValueError("step must be a nonnegative integer")
    if int(accum_steps) != accum_steps or accum_steps < 1:
        raise ValueError("accum_steps must be a positive integer")
    if int(microbatch_index) != microbatch_index or not 0 <= microbatch_index < accum_steps:
        raise ValueError("microbatch_index must be in [0, accum_steps)")
    if isinstance(layers, nn.Module):
        layers = [m for m in layers.modules() if isinstance(m, (STACRLinear, AdaptiveLinear))]
    for layer in layers:
        if isinstance(layer, AdaptiveLinear):
            layer.set_runtime_state(optimizer_step=step, microbatch_index=microbatch_index, accum_steps=accum_steps)
        else:
            layer.set_step(step)
