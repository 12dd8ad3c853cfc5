"""Read-only measurement mode: compressed gradients on, stochastic layers off, state restored afterwards.

Inside the context every compressed layer behaves as in training (so backward goes through the
factor-native path) while the rest of the model is in eval mode; bases, counters, controllers and
configs are put back exactly as they were on exit.  Parity: stacr/diagnostics.py:25-87 of the
reference project.
"""

from __future__ import annotations

import copy
from contextlib import contextmanager

import torch

from .adaptive import STACRLinear as AdaptiveLinear
from .adaptive_checkpointing import get_global_recomputation_guard
from .layers import STACRLinear


def _deep_clone(value):
    if isinstance(value, torch.Tensor):
        return value.detach().clone()
    if isinstance(value, dict):
        return {k: _deep_clone(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_deep_clone(v) for v in value)
    return value


class _LayerMemo:
    """Everything a diagnostic forward could disturb on one layer."""

    def __init__(self, layer):
        self.layer = layer
        # the basis tensor is immutable by contract: keep the object itself, clone the scalars
        self.buffers = {k: (t if k == "basis" or t is None else t.detach().clone()) for k, t in layer._buffers.items()}
        if isinstance(layer, AdaptiveLinear):
            self.config_obj, self.config_copy = layer.config, copy.deepcopy(layer.config)
            self.state = _deep_clone(layer.layer_state)
            self.host = (layer._h_init, layer._h_forward_calls, layer._cached_step_basis)
        else:
            self.knobs = (layer.freeze_after_warmup, layer.warmup_steps)
            self.host = (layer._h_step, layer._h_last, layer._h_ready)

    def restore(self):
        layer = self.layer
        for key, tensor in self.buffers.items():
            setattr(layer, key, tensor)
        if isinstance(layer, AdaptiveLinear):
            self.config_obj.__dict__.clear()
            self.config_obj.__dict__.update(self.config_copy.__dict__)
            layer.config = self.config_obj
            layer.layer_state.clear()
            layer.layer_state.update(self.state)
            layer._h_init, layer._h_forward_calls, layer._cached_step_basis = self.host
        else:
            layer.freeze_after_warmup, layer.warmup_steps = self.knobs
            layer._h_step, layer._h_last, layer._h_ready = self.host


@contextmanager
def compression_diagnostics(model):
    """Run forwards/backwards that use compression but leave no trace in compression state."""
    layers = [m for m in model.modules() if isinstance(m, (STACRLinear, AdaptiveLinear))]
    for layer in layers:
        if isinstance(layer, AdaptiveLinear) and layer.config.residual_mode != "sparse_only" and not layer.basis_initialized:
            raise ValueError("Initialize adaptive bases with a training forward before computing fidelity")
    modes = {m: m.training for m in model.modules()}
    memos = [_LayerMemo(layer) for layer in layers]
    try:
        model.eval()
        for layer in layers:
            layer.training = True
            if isinstance(layer, STACRLinear):
                layer._sync_host()
                layer.freeze_after_warmup, layer.warmup_steps = True, 0
        with get_global_recomputation_guard().recomputation_context():
            yield
    finally:
        for memo in memos:
            memo.restore()
        for m, flag in modes.items():
            m.training = flag
