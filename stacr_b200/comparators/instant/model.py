"""Model surgery of the INSTANT comparator (parity: comparators/instant/model.py)."""

from __future__ import annotations

import re

import torch.nn as nn

from .custom_op import InstantLinear

_SKIP = {
    "bert": ("classifier", "embeddings", "pooler"),
    "distilbert": ("classifier", "embeddings", "pre_classifier"),
    "gpt2": ("lm_head", "wte", "wpe", "ln_f"),
}
_BLOCK_PATTERNS = (r"encoder\.layer\.(\d+)\.", r"transformer\.layer\.(\d+)\.", r"transformer\.h\.(\d+)\.",
                   r"layers\.(\d+)\.", r"\bh\.(\d+)\.")
_HEAD_NAMES = ("classifier", "pre_classifier", "lm_head", "ln_f", "score", "embed_out", "final_layer_norm")


def _family(model_name) -> str:
    name = (model_name or "").lower()
    for fam in ("distilbert", "bert", "gpt2"):
        if fam in name:
            return fam
    return "bert"


def _skip_layer(name: str, model_name) -> bool:
    return any(part in name for part in _SKIP[_family(model_name)])


def _block_index(param_name: str):
    for pat in _BLOCK_PATTERNS:
        m = re.search(pat, param_name)
        if m:
            return int(m.group(1))
    return None


def freeze_layers(model: nn.Module, n_last_layers: int, model_name=None) -> None:
    """Train only the last ``n_last_layers`` transformer blocks and the head; 0 leaves everything trainable."""
    if not n_last_layers:
        return
    indices = {i for i in (_block_index(n) for n, _ in model.named_parameters()) if i is not None}
    first_trainable = (max(indices) + 1 if indices else 0) - int(n_last_layers)
    for name, param in model.named_parameters():
        idx = _block_index(name)
        if idx is not None:
            param.requires_grad = idx >= first_trainable
        else:
            param.requires_grad = any(h in name for h in _HEAD_NAMES)


freeze_bert_layers = freeze_layers


def convert_conv1d_to_linear(model: nn.Module) -> nn.Module:
    """Replace ``transformers`` ``Conv1D`` modules (weight ``[in, out]``) by ``nn.Linear``; the in-tree models need none."""
    try:
        from transformers.pytorch_utils import Conv1D
    except Exception:
        return model
    for name, module in list(model.named_modules()):
        if isinstance(module, Conv1D):
            fan_in, fan_out = module.weight.shape
            lin = nn.Linear(fan_in, fan_out, bias=module.bias is not None, device=module.weight.device, dtype=module.weight.dtype)
            lin.weight.data.copy_(module.weight.data.t())
            if module.bias is not None:
                lin.bias.data.copy_(module.bias.data)
            parent_name, _, leaf = name.rpartition(".")
            setattr(model.get_submodule(parent_name) if parent_name else model, leaf, lin)
    return model


def get_svd_layers(model: nn.Module, model_name=None) -> list[str]:
    """Names of trainable ``nn.Linear`` modules outside embeddings and heads."""
    names = []
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear) and any(p.requires_grad for p in module.parameters()) and not _skip_layer(name, model_name):
            names.append(name)
    return names


def update_compression(model: nn.Module, p_dict: dict, q_dict: dict) -> nn.Module:
    for name, module in model.named_modules():
        if isinstance(module, InstantLinear) and name in p_dict and name in q_dict:
            module.CompressionTensor_x = p_dict[name].detach()
            module.CompressionTensor_gy = q_dict[name].detach()
    return model


def _set_active(model: nn.Module, flag: bool) -> nn.Module:
    for module in model.modules():
        if isinstance(module, InstantLinear):
            module.activate = flag
    return model


def enable_compression(model: nn.Module) -> nn.Module:
    return _set_active(model, True)


def disable_compression(model: nn.Module) -> nn.Module:
    return _set_active(model, False)


def print_status(model: nn.Module) -> None:
    for name, param in model.named_parameters():
        print(f"{'trainable' if param.requires_grad else 'frozen':9s} {name}")


def add_activate_to_module() -> None:
    """Kept for scripts that call it: the on/off switch is a class attribute of ``InstantLinear`` here, toggled per model by
    :func:`enable_compression` / :func:`disable_compression`, so ``nn.Module`` is not patched."""
    return None


def add_compression_tensor_to_module() -> None:
    """Kept for scripts that call it: the two subspaces are attributes of ``InstantLinear``, installed by :func:`update_compression`."""
    return None
