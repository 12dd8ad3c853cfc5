"""Calibration of the token subspaces (parity: comparators/instant/callback.py).

The reference hangs its calibration on ``transformers.Trainer`` callbacks and module-level dictionaries; here it is
one object that owns its hooks and state, usable from any loop: ``Calibrator(model, names).run(batches, loss_fn)``.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .model import disable_compression, enable_compression, update_compression
from .svd import energy_basis


class Calibrator:
    def __init__(self, model: nn.Module, layer_names, var: float = 0.95, over_sampling: int = 7):
        self.model, self.names = model, list(layer_names)
        self.var, self.over_sampling = float(var), int(over_sampling)
        self.gram_x: dict[str, torch.Tensor] = {}
        self.gram_g: dict[str, torch.Tensor] = {}
        self.P: dict[str, torch.Tensor] = {}
        self.Q: dict[str, torch.Tensor] = {}
        self._handles: list = []

    @staticmethod
    def _token_gram(t: torch.Tensor) -> torch.Tensor:
        if t.dim() != 3:
            raise ValueError(f"calibration expects [batch, tokens, features], got {tuple(t.shape)}")
        t = t.detach().float()
        return torch.einsum("bsf,btf->st", t, t) / t.shape[0]

    def _accumulate(self, store, name, t):
        g = self._token_gram(t)
        if name in store and store[name].shape == g.shape:
            store[name] += g
        else:
            store[name] = g

    def register_hooks(self) -> None:
        for name in self.names:
            module = self.model.get_submodule(name)
            self._handles.append(module.register_forward_hook(
                lambda m, inp, out, name=name: self._accumulate(self.gram_x, name, inp[0])))
            self._handles.append(module.register_full_backward_hook(
                lambda m, gin, gout, name=name: self._accumulate(self.gram_g, name, gout[0])))

    def unregister_hooks(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles.clear()
        self.gram_x.clear()
        self.gram_g.clear()

    def solve(self) -> None:
        for name in self.names:
            if name in self.gram_x and name in self.gram_g:
                self.P[name] = energy_basis(self.gram_x[name], self.var, self.over_sampling)
                self.Q[name] = energy_basis(self.gram_g[name], self.var, self.over_sampling)

    def run(self, batches, loss_of_batch) -> dict:
        """Uncompressed forward/backward over ``batches`` (gradients discarded), then install fresh subspaces.

        ``loss_of_batch(model, batch)`` returns the scalar loss.  Returns ``{layer: (k_x, k_g)}``.
        """
        was_training = self.model.training
        self.model.train()
        disable_compression(self.model)
        self.register_hooks()
        try:
            for batch in batches:
                loss_of_batch(self.model, batch).backward()
                self.model.zero_grad(set_to_none=True)
            self.solve()
        finally:
            self.unregister_hooks()
            enable_compression(self.model)
            self.model.train(was_training)
        update_compression(self.model, self.P, self.Q)
        return {n: (int(self.P[n].shape[1]), int(self.Q[n].shape[1])) for n in self.P}


# ------------------------------------------------------------------------------ module-level form
# Scripts written against the upstream layout register hooks once per calibration window through module functions and
# read the accumulated Gram matrices from module dictionaries; these wrap one shared Calibrator.
_ACTIVE: dict = {"calibrator": None}
layer_inputs: dict = {}
layer_gradients: dict = {}
P_dict: dict = {}
Q_dict: dict = {}


def register_hooks(model: nn.Module, model_name=None, var: float = 0.95, over_sampling: int = 7) -> Calibrator:
    from .model import get_svd_layers

    unregister_hooks()
    calib = Calibrator(model, get_svd_layers(model, model_name), var=var, over_sampling=over_sampling)
    calib.gram_x, calib.gram_g, calib.P, calib.Q = layer_inputs, layer_gradients, P_dict, Q_dict
    calib.register_hooks()
    _ACTIVE["calibrator"] = calib
    return calib


def unregister_hooks() -> None:
    calib = _ACTIVE.get("calibrator")
    if calib is not None:
        calib.unregister_hooks()
    _ACTIVE["calibrator"] = None
    for store in (layer_inputs, layer_gradients, P_dict, Q_dict):
        store.clear()


def save_input_hook(name, module, input, output) -> None:
    """Accumulate the batch-averaged token Gram matrix of a layer input (the forward-hook body)."""
    Calibrator._accumulate(_ACTIVE.get("calibrator") or Calibrator(module, []), layer_inputs, name, input[0])


def save_grad_hook(name, module, grad_input, grad_output) -> None:
    """Accumulate the batch-averaged token Gram matrix of a layer's output gradient (the backward-hook body)."""
    Calibrator._accumulate(_ACTIVE.get("calibrator") or Calibrator(module, []), layer_gradients, name, grad_output[0])


class CustomLoggingCallback:
    """Recalibration on a step schedule for loops that call ``on_step_begin(step, model, batches, loss_of_batch)``.

    The upstream class is a ``transformers.TrainerCallback``; this one has no framework dependency and the in-tree
    training scripts (``_loop.run``) inline the same schedule.
    """

    def __init__(self, args):
        self.args, self.calibrator = args, None

    def on_step_begin(self, step: int, model: nn.Module, batches, loss_of_batch, model_name=None):
        if not getattr(self.args, "compress", False) or step % max(int(getattr(self.args, "calib_iter", 50)), 1):
            return None
        if self.calibrator is None:
            from .model import get_svd_layers

            self.calibrator = Calibrator(model, get_svd_layers(model, model_name), var=getattr(self.args, "var", 0.95),
                                         over_sampling=getattr(self.args, "over_sampling", 7))
        return self.calibrator.run(batches, loss_of_batch)
