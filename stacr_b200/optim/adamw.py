"""AdamW with fp32 or 8-bit block-wise moments, stepped by one multi-tensor kernel launch per group.

On CUDA the update runs in ``csrc/optim.cu``; on CPU the same arithmetic is done with framework
ops (the 8-bit code path included, so the codec is testable without a GPU).  ``AdamW8bit``
replaces the external 8-bit optimizer the reference builds through
stacr/protocols/baselines/bnb_optimizer.py:61-176 (tensors below ``min_8bit_size`` elements keep
fp32 moments, block size 256).
"""

from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

BLOCK = 256


# ----------------------------------------------------------------------------- 8-bit codec (framework ops)
def encode_first_moment(m: torch.Tensor):
    """Signed square-root companding, per 256-element block.  Returns ``(uint8 codes, fp32 absmax)``."""
    flat = m.reshape(-1).float()
    pad = (-flat.numel()) % BLOCK
    blocks = torch.nn.functional.pad(flat, (0, pad)).view(-1, BLOCK)
    amax = blocks.abs().amax(1)
    safe = amax.clamp_min(1e-38)[:, None]
    s = torch.sqrt((blocks.abs() / safe).clamp_max(1.0)) * torch.sign(blocks)
    codes = (128 + torch.round(s * 127)).to(torch.uint8)
    codes = torch.where(amax[:, None] > 0, codes, torch.full_like(codes, 128))
    return codes.view(-1)[: flat.numel()], amax


def decode_first_moment(codes: torch.Tensor, amax: torch.Tensor) -> torch.Tensor:
    n = codes.numel()
    pad = (-n) % BLOCK
    c = torch.nn.functional.pad(codes.float(), (0, pad), value=128.0).view(-1, BLOCK)
    s = (c - 128.0) / 127.0
    return (torch.sign(s) * s * s * amax[:, None]).view(-1)[:n]


def encode_second_moment(v: torch.Tensor):
    """Unsigned fourth-root companding, per 256-element block."""
    flat = v.reshape(-1).float()
    pad = (-flat.numel()) % BLOCK
    blocks = torch.nn.functional.pad(flat, (0, pad)).view(-1, BLOCK)
    amax = blocks.amax(1)
    safe = amax.clamp_min(1e-38)[:, None]
    codes = torch.round((blocks / safe).clamp(0, 1).pow(0.25) * 255).to(torch.uint8)
    codes = torch.where(amax[:, None] > 0, codes, torch.zeros_like(codes))
    return codes.view(-1)[: flat.numel()], amax


def decode_second_moment(codes: torch.Tensor, amax: torch.Tensor) -> torch.Tensor:
    n = codes.numel()
    pad = (-n) % BLOCK
    c = torch.nn.functional.pad(codes.float(), (0, pad)).view(-1, BLOCK) / 255.0
    return (c.pow(4) * amax[:, None]).view(-1)[:n]


_DESC = np.dtype(
    [("param", "<u8"), ("grad", "<u8"), ("m", "<u8"), ("v", "<u8"), ("shadow", "<u8"), ("m8", "<u8"), ("v8", "<u8"),
     ("m_absmax", "<u8"), ("v_absmax", "<u8"), ("numel", "<i8"), ("shadow_mc", "<u8")]
)
_CHUNK = np.dtype([("tensor", "<i4"), ("pad", "<i4"), ("offset", "<i8")])


class AdamW(torch.optim.Optimizer):
    """Decoupled-weight-decay Adam.  ``eight_bit=True`` keeps both moments as block-wise 8-bit codes.

    ``bf16_shadow=True`` additionally maintains ``param._bf16_shadow``, a bf16 copy refreshed inside
    the update kernel so that bf16 forwards need no per-step cast of the master weights.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, *, eight_bit=False,
                 min_8bit_size=4096, bf16_shadow=False, shard=None):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid AdamW hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.eight_bit, self.min_8bit_size, self.bf16_shadow = bool(eight_bit), int(min_8bit_size), bool(bf16_shadow)
        # ``shard``: a ``parallel.zero.ShardedGradSync``.  Parameters it shards are updated only over the element ranges this
        # rank owns; their bf16 copies belong to it (views of one flat buffer) and it publishes the update to the other ranks.
        self.shard = shard
        # CUDA-graph mode (see ``enable_graph_mode``): hyper-parameters and bias corrections live in device memory
        self._graph_hyper = None
        self._graph_pins: list = []
        self._tables: dict[int, dict] = {}
        self.kernel_launches = 0

    # ------------------------------------------------------------------ state
    def _init_state(self, p: torch.Tensor) -> dict:
        st = self.state[p]
        if st:
            return st
        st["step"] = 0
        use8 = self.eight_bit and p.numel() >= self.min_8bit_size
        st["eight_bit"] = use8
        if use8:
            nblk = (p.numel() + BLOCK - 1) // BLOCK
            st["m8"] = torch.full((p.numel(),), 128, dtype=torch.uint8, device=p.device)
            st["v8"] = torch.zeros(p.numel(), dtype=torch.uint8, device=p.device)
            st["m_absmax"] = torch.zeros(nblk, dtype=torch.float32, device=p.device)
            st["v_absmax"] = torch.zeros(nblk, dtype=torch.float32, device=p.device)
        else:
            st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.contiguous_format)
        if self.bf16_shadow and p.is_cuda and getattr(p, "_bf16_shadow", None) is None:
            p._bf16_shadow = p.detach().to(torch.bfloat16)
            p._bf16_shadow_version = p._version
        return st

    # ------------------------------------------------------------------ CUDA-graph mode
    def enable_graph_mode(self, device) -> None:
        """Prepare the optimizer for a step that is captured once and replayed from a CUDA graph.

        Kernel arguments are frozen at capture time, so the per-step scalars (learning rate, bias corrections, gradient
        scale) move to a small device array; :meth:`graph_pre_step` advances the step counters on the host and refreshes
        that array with one asynchronous copy in front of each replay.  Inside the captured ``step()`` nothing is counted.
        """
        n = len(self.param_groups)
        self._graph_hyper = {"dev": torch.zeros(n, 8, dtype=torch.float32, device=device),
                             "host": torch.zeros(n, 8, dtype=torch.float32).pin_memory(), "scale": 1.0}

    def graph_pre_step(self, grad_scale: float = 1.0) -> None:
        """Advance the step counters and upload this step's scalars (call before capture and before every replay)."""
        gh = self._graph_hyper
        for gi, group in enumerate(self.param_groups):
            step = None
            for p in group["params"]:
                if p.requires_grad:
                    st = self._init_state(p)
                    st["step"] += 1
                    step = st["step"]
            if step is None:
                continue
            b1, b2 = group["betas"]
            gh["host"][gi] = torch.tensor([group["lr"], b1, b2, group["eps"], group["weight_decay"], 1 - b1 ** step, 1 - b2 ** step, grad_scale])
        gh["dev"].copy_(gh["host"], non_blocking=True)

    def _ranges(self, p: torch.Tensor):
        """Element ranges of ``p`` this rank updates: everything, unless a sharding synchroniser owns the partition."""
        if self.shard is not None and self.shard.is_sharded(p):
            return self.shard.owned_ranges(p)
        return [(0, p.numel())]

    def close(self) -> None:
        """Detach the bf16 shadows from the parameters (call before handing the model to another optimizer)."""
        for group in self.param_groups:
            for p in group["params"]:
                for attr in ("_bf16_shadow", "_bf16_shadow_version"):
                    if hasattr(p, attr):
                        delattr(p, attr)

    def state_bytes(self) -> int:
        total = 0
        for st in self.state.values():
            total += sum(t.numel() * t.element_size() for t in st.values() if torch.is_tensor(t))
        return total

    # ------------------------------------------------------------------ CPU / reference arithmetic
    @staticmethod
    def _reference_update(p, g, st, lr, b1, b2, eps, wd, bias1, bias2):
        if st["eight_bit"]:
            m = decode_first_moment(st["m8"], st["m_absmax"]).view_as(p)
            v = decode_second_moment(st["v8"], st["v_absmax"]).view_as(p)
        else:
            m, v = st["exp_avg"], st["exp_avg_sq"]
        m = b1 * m + (1 - b1) * g
        v = b2 * v + (1 - b2) * g * g
        p.mul_(1 - lr * wd)
        p.addcdiv_(m / bias1, (v / bias2).sqrt() + eps, value=-lr)
        if st["eight_bit"]:
            st["m8"], st["m_absmax"] = encode_first_moment(m)
            st["v8"], st["v_absmax"] = encode_second_moment(v)
        else:
            st["exp_avg"], st["exp_avg_sq"] = m, v

    # ------------------------------------------------------------------ kernel tables
    def _launch_group(self, gi: int, group: dict, plist: list, grad_scale: float) -> None:
        from ..ops import _lib

        lib = _lib.load()
        dev = plist[0].device
        cache = self._tables.get(gi)
        ranges = [self._ranges(p) for p in plist]
        sig = tuple((p.data_ptr(), p.numel(), tuple(r)) for p, r in zip(plist, ranges))
        if cache is None or cache["sig"] != sig:
            chunk = lib.sb_optim_chunk()
            rows = []
            for ti, (p, rs) in enumerate(zip(plist, ranges)):
                for a, b in rs:
                    assert a % chunk == 0, "an owned range must start on a chunk boundary"
                    rows += [(ti, 0, off) for off in range(a, b, chunk)]
            if not rows:
                self._tables[gi] = {"sig": sig, "n_chunks": 0}
                return
            chunks = np.array(rows, dtype=_CHUNK)
            cache = {
                "sig": sig,
                "n_chunks": len(rows),
                "chunks": torch.from_numpy(chunks.view(np.uint8).copy()).to(dev),
                # two pinned staging tables, each guarded by an event recorded behind its upload: the host never
                # rewrites a table whose copy to the device may still be pending
                "host": [torch.zeros(len(plist) * _DESC.itemsize, dtype=torch.uint8, pin_memory=True) for _ in range(2)],
                "events": [None, None],
                "turn": 0,
                "last": None,
                "dev": torch.empty(len(plist) * _DESC.itemsize, dtype=torch.uint8, device=dev),
            }
            assert lib.sb_tensor_desc_size() == _DESC.itemsize and lib.sb_chunk_desc_size() == _CHUNK.itemsize
            self._tables[gi] = cache
        if cache["n_chunks"] == 0:
            return
        table = np.empty(len(plist), dtype=_DESC)
        for ti, p in enumerate(plist):
            st = self.state[p]
            ptr = lambda t: 0 if t is None else t.data_ptr()
            table[ti] = (
                p.data_ptr(), p.grad.data_ptr(), ptr(st.get("exp_avg")), ptr(st.get("exp_avg_sq")),
                ptr(getattr(p, "_bf16_shadow", None)), ptr(st.get("m8")), ptr(st.get("v8")), ptr(st.get("m_absmax")),
                ptr(st.get("v_absmax")), p.numel(), int(getattr(p, "_bf16_shadow_mc", 0) or 0),
            )
        blob = table.tobytes()
        capturing = torch.cuda.is_current_stream_capturing()
        if capturing:
            # the copy becomes a node of the graph and is replayed with it: it needs a pinned source of its own that stays
            # untouched for the life of the graph (no event may be waited on while a stream is capturing)
            pin = torch.empty(len(blob), dtype=torch.uint8).pin_memory()
            pin.numpy()[:] = np.frombuffer(blob, dtype=np.uint8)
            self._graph_pins.append(pin)
            cache["dev"].copy_(pin, non_blocking=True)
            cache["last"] = None
        elif blob != cache["last"]:
            # the pointers changed (gradients are reallocated when they are dropped between steps): upload through the
            # staging table whose previous upload has certainly finished
            turn = cache["turn"]
            if cache["events"][turn] is not None:
                cache["events"][turn].synchronize()
            cache["host"][turn].numpy()[:] = np.frombuffer(blob, dtype=np.uint8)
            cache["dev"].copy_(cache["host"][turn], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            cache["events"][turn] = ev
            cache["turn"] = turn ^ 1
            cache["last"] = blob
        step = max(1, self.state[plist[0]]["step"])
        b1, b2 = group["betas"]
        hyper = None if self._graph_hyper is None else self._graph_hyper["dev"][gi]
        rc = lib.sb_adamw_step(
            _lib.ptr(cache["dev"]), _lib.ptr(cache["chunks"]), ctypes.c_int(cache["n_chunks"]), ctypes.c_int(int(self.eight_bit)),
            ctypes.c_float(group["lr"]), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(group["eps"]),
            ctypes.c_float(group["weight_decay"]), ctypes.c_float(1 - b1 ** step), ctypes.c_float(1 - b2 ** step),
            ctypes.c_float(grad_scale), _lib.ptr(hyper), _lib.stream_ptr(),
        )
        _lib.check_rc(rc, "sb_adamw_step")
        self.kernel_launches += 1
        if self.bf16_shadow:
            for p in plist:      # the kernel refreshed master and shadow together through raw pointers
                p._bf16_shadow_version = p._version

    @torch.no_grad()
    def step(self, closure=None, grad_scale: float = 1.0):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            fast, slow = [], []
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AdamW does not support sparse gradients")
                st = self._init_state(p)
                if self._graph_hyper is None:
                    st["step"] += 1          # in graph mode the counters are advanced by graph_pre_step()
                ok = p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and p.is_contiguous() and p.grad.is_contiguous()
                (fast if ok else slow).append(p)
            if fast:
                steps = {self.state[p]["step"] for p in fast}
                if len(steps) == 1:
                    self._launch_group(gi, group, fast, grad_scale)
                else:
                    slow += fast
            b1, b2 = group["betas"]
            for p in slow:
                st = self.state[p]
                full = [(0, p.numel())]
                ranges = self._ranges(p)
                if ranges == full:
                    g = p.grad.float() * grad_scale
                    work = p.data.float() if p.dtype != torch.float32 else p.data
                    self._reference_update(work, g, st, group["lr"], b1, b2, group["eps"], group["weight_decay"],
                                           1 - b1 ** st["step"], 1 - b2 ** st["step"])
                    if work is not p.data:
                        p.data.copy_(work)
                else:
                    self._reference_update_ranges(p, st, ranges, group, grad_scale)
                if hasattr(p, "_bf16_shadow"):
                    p._bf16_shadow.copy_(p.data)
                    p._bf16_shadow_version = p._version
        if self.shard is not None:
            self.shard.publish_updates()
        return loss

    def _reference_update_ranges(self, p, st, ranges, group, grad_scale) -> None:
        """The framework-op update restricted to chunk-aligned element ranges of a contiguous parameter (sharded optimizer)."""
        b1, b2 = group["betas"]
        flat_p, flat_g = p.data.view(-1), p.grad.reshape(-1)
        for a, b in ranges:
            sub = {"eight_bit": st["eight_bit"]}
            if st["eight_bit"]:
                qa, qb = a // BLOCK, (b + BLOCK - 1) // BLOCK
                sub.update(m8=st["m8"][a:b], v8=st["v8"][a:b], m_absmax=st["m_absmax"][qa:qb], v_absmax=st["v_absmax"][qa:qb])
            else:
                sub.update(exp_avg=st["exp_avg"].view(-1)[a:b], exp_avg_sq=st["exp_avg_sq"].view(-1)[a:b])
            work = flat_p[a:b].float() if p.dtype != torch.float32 else flat_p[a:b]
            self._reference_update(work, flat_g[a:b].float() * grad_scale, sub, group["lr"], b1, b2, group["eps"], group["weight_decay"],
                                   1 - b1 ** st["step"], 1 - b2 ** st["step"])
            if work is not flat_p[a:b]:
                flat_p[a:b].copy_(work)
            if st["eight_bit"]:
                st["m8"][a:b], st["v8"][a:b] = sub["m8"], sub["v8"]
                st["m_absmax"][qa:qb], st["v_absmax"][qa:qb] = sub["m_absmax"], sub["v_absmax"]
            else:
                st["exp_avg"].view(-1)[a:b], st["exp_avg_sq"].view(-1)[a:b] = sub["exp_avg"], sub["exp_avg_sq"]


class AdamW8bit(AdamW):
    """AdamW with 8-bit block-wise moments (256-element blocks, fp32 absmax per block)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, min_8bit_size=4096, **kw):
        super().__init__(params, lr, betas, eps, weight_decay, eight_bit=True, min_8bit_size=min_8bit_size, **kw)
