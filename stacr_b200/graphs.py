"""A whole training step as one CUDA graph.

The compressed layers launch a few dozen small kernels each; with well over a hundred wrapped projections (GPT-2 large
with the attention surface: 144) the host cannot issue launches as fast as the GPU retires them and the step becomes
launch-bound.  ``GraphedStep`` captures forward, backward, gradient synchronisation and the optimizer update of one step
once and replays it with a single launch.

What makes a step replayable here:

* inputs live in static buffers that are overwritten before each replay; the loss comes back in a static tensor;
* the optimizer reads its per-step scalars (learning rate, bias corrections) from device memory (``AdamW.enable_graph_mode``);
* a tracked basis is *rebound* to a new tensor by every update; replays read the basis from the storage it had at capture
  time, so the capture ends by copying every new version (and its cached bf16 views) back into the old storage;
* host-side schedules (``set_step``) are frozen at capture: a graph is valid for a phase in which the same kernels run
  every step (basis updated every step, residual kept or dropped).  ``valid_for(step)`` tells the caller when the phase
  ends (``turbo_after_step``, ``freeze_after_warmup``); re-capture or fall back to the eager step then.

Device-to-host reads, allocator growth and event waits must not happen inside the step function.
"""

from __future__ import annotations

from typing import Callable, Iterable, Optional, Sequence

import torch

from . import layers as _layers


class GraphedStep:
    """Capture ``step_fn(*inputs) -> loss`` once and replay it.

    ``step_fn`` must do everything of one optimizer step except reading results on the host: ``set_step`` on the wrapped
    layers is done here (``layers``), ``optimizer.step()`` is called inside ``step_fn`` with the optimizer given here.
    ``example_inputs`` fix the shapes; ``__call__`` copies new inputs into the static buffers and returns the static loss.
    """

    def __init__(self, step_fn: Callable, example_inputs: Sequence[torch.Tensor], *, optimizer=None, layers: Iterable = (),
                 first_step: int = 0, warmup: int = 3, prep_inputs: Optional[Sequence[Sequence[torch.Tensor]]] = None):
        self.step_fn = step_fn
        self.optimizer = optimizer
        self.layers = list(layers)
        self.step = int(first_step)
        self.static_inputs = [t.clone() for t in example_inputs]
        dev = self.static_inputs[0].device
        if optimizer is not None and hasattr(optimizer, "enable_graph_mode"):
            optimizer.enable_graph_mode(dev)
        # eager warm-up on a side stream (lazy initialisation, caches, the allocator's pools), as capture requires
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        # ``prep_inputs``: the inputs of the warm-up steps and of the captured step, in order (each a sequence like
        # ``example_inputs``).  These are real training steps; feeding them the next batches of the data stream, rather than
        # the example batch every time, keeps the run on the trajectory an eager loop would have taken.
        prep = [list(p) for p in (prep_inputs or [])]
        with torch.cuda.stream(side):
            for k in range(max(1, warmup)):
                if k < len(prep):
                    for static, new in zip(self.static_inputs, prep[k]):
                        static.copy_(new)
                self._pre()
                out = step_fn(*self.static_inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        del out
        self.graph = torch.cuda.CUDAGraph()
        if len(prep) > max(1, warmup):
            for static, new in zip(self.static_inputs, prep[max(1, warmup)]):
                static.copy_(new)
            torch.cuda.synchronize(dev)
        self._pre()
        _layers.GRAPH_BASIS_PAIRS = pairs = []
        try:
            with torch.cuda.graph(self.graph, capture_error_mode="relaxed"):
                self.static_loss = step_fn(*self.static_inputs)
                self._copy_back(pairs)
        finally:
            _layers.GRAPH_BASIS_PAIRS = None
        self.basis_pairs = len(pairs)
        self.replays = 0

    def _pre(self) -> None:
        for layer in self.layers:
            if hasattr(layer, "_h_step"):
                layer._sync_host()
                layer._h_step = self.step          # host mirror only: no device fill per layer per step (see sync_state)
            elif hasattr(layer, "set_step"):
                layer.set_step(self.step)
        if self.optimizer is not None and hasattr(self.optimizer, "graph_pre_step"):
            self.optimizer.graph_pre_step()
        self.step += 1

    @staticmethod
    @torch.no_grad()
    def _copy_back(pairs) -> None:
        dst, src = [], []
        for old, new in pairs:
            if old is new or old.shape != new.shape or old.dtype != new.dtype:
                continue
            dst.append(old)
            src.append(new)
            ov, nv = getattr(old, "_sb_views", None), getattr(new, "_sb_views", None)
            if ov is not None and nv is not None:
                dst += [ov[0], ov[1]]
                src += [nv[0], nv[1]]
        if dst:
            torch._foreach_copy_(dst, src)

    def valid_for(self, step: Optional[int] = None) -> bool:
        """False once a wrapped layer's schedule changes what a step does (turbo phase, frozen basis)."""
        step = self.step if step is None else step
        for layer in self.layers:
            turbo = getattr(layer, "turbo_after_step", None)
            if turbo is not None and step >= int(turbo):
                return False
            if getattr(layer, "freeze_after_warmup", False) and step >= int(getattr(layer, "warmup_steps", 0)):
                return False
        return True

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        for static, new in zip(self.static_inputs, inputs):
            if new is not static:
                static.copy_(new, non_blocking=True)
        self._pre()
        self.graph.replay()
        self.replays += 1
        return self.static_loss

    def sync_state(self) -> None:
        """Bring the layers' device-side step counters up to date (they are not advanced by replays); call before ``state_dict``."""
        for layer in self.layers:
            if hasattr(layer, "_step"):
                layer._step.fill_(max(0, self.step - 1))
                layer._last_update_step.fill_(max(0, self.step - 1))
