"""Search-style measurements built on ``common.run_config``: the largest batch or sequence that trains, a single guarded
cell, and paired gradients of one model.  The per-grid entry modules bind these to their models and arms.

Parity: the ``one``/``maxlen``/``maxbatch``/``largest_fitting``/``grads`` helpers of experiments/benchmarks/
sequence_length.py:60-170, large_models.py, capacity_search.py:25-60 and single_model_fidelity.py:40-53.
"""

from __future__ import annotations

from typing import Iterable, Optional

import torch

from . import common


def complement(k: int):
    """Predicate selecting the blocks a 1-in-``k`` checkpointing plan leaves alone (``index % k != 0``)."""
    return lambda index, _k=int(k): index % _k != 0


def one(model_id: str, tag: str, method: str, extra: dict, bs: int, seq: int, seed: int = 42, baseline_peak=None, out=None, **run_kw) -> Optional[dict]:
    """Run one cell; an out-of-memory or failed cell is recorded and returns ``None`` so that a search can stop there."""
    try:
        rec = common.run_config(method, seed, model_id=model_id, bs=bs, seq=seq, baseline_peak_bytes=baseline_peak, **{**run_kw, **extra})
        rec["tag"] = tag
    except torch.cuda.OutOfMemoryError:
        rec = {"tag": tag, "method": method, "model": model_id, "bs": bs, "seq": seq, "seed": seed, "status": "OOM", "fits": False}
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001  (a failed cell must not end the sweep)
        rec = {"tag": tag, "method": method, "model": model_id, "bs": bs, "seq": seq, "seed": seed, "status": "error", "fits": False,
               "error": f"{type(exc).__name__}: {exc}"[:300]}
    if out is not None and common._RECORDER is None:
        common.emit(rec, out)
    return rec if rec.get("status", "ok") == "ok" else None


def _ascend(values: Iterable[int], run) -> Optional[dict]:
    best = None
    for value in values:
        rec = run(value)
        if rec is None:
            break
        best = rec
    return best


def maxlen(model_id: str, method: str, extra: dict, lengths: Iterable[int], bs: int = 1, out=None, tag: str = "maxlen", **run_kw) -> Optional[dict]:
    """The longest sequence in ``lengths`` (ascending) that trains at batch ``bs``; the row of that run, or ``None``."""
    return _ascend(lengths, lambda seq: one(model_id, f"{tag}/s{seq}", method, extra, bs, seq, out=out, **run_kw))


def maxbatch(model_id: str, method: str, extra: dict, batches: Iterable[int], seq: int = 4096, out=None, tag: str = "maxbatch", **run_kw) -> Optional[dict]:
    """The largest batch in ``batches`` (ascending) that trains at sequence length ``seq``."""
    return _ascend(batches, lambda bs: one(model_id, f"{tag}/b{bs}", method, extra, bs, seq, out=out, **run_kw))


def largest_fitting(model_id: str, seq: int, dtype, lo: int, hi: int, method: str, cfg: Optional[dict], out=None, tag: str = "capacity", **run_kw) -> Optional[dict]:
    """Batch sizes ``lo..hi`` in turn until one fails; returns the last row that fitted (each row carries ``fits``)."""
    opts = {"steps": 12, "measure_from": 5, "eval_batches": 2, "model_dtype": dtype, **run_kw}
    opts["measure_from"] = min(opts["measure_from"], max(0, opts["steps"] - 1))

    def run(bs):
        rec = one(model_id, tag, method, {"stacr_cfg": cfg} if cfg else {}, bs, seq, out=None, **opts)
        row = dict(rec, fits=True) if rec else {"tag": tag, "method": method, "bs": bs, "seq": seq, "fits": False}
        if out is not None and common._RECORDER is None:
            common.emit(row, out)
        return rec

    return _ascend(range(int(lo), int(hi) + 1), run)


def sweep(model_id: str, arms, lengths: Iterable[int], bs: int = 1, seeds=(42,), out=None, tag: str = "sweep", **run_kw) -> list:
    """Every arm at every length and seed; savings are reported against the first arm's peak at the same length."""
    rows = []
    for seq in lengths:
        base = None
        for method, extra in arms:
            for seed in seeds:
                rec = one(model_id, f"{tag}/s{seq}", method, extra, bs, seq, seed, base, out, **run_kw)
                if rec is not None:
                    if base is None:
                        base = rec.get("peak_bytes")
                    rows.append(rec)
    return rows


def grads(model, batch, seed: int, amp: bool = False):
    """``({name: fp32 gradient}, loss)`` of one forward/backward with the RNG seeded, so that two calls see the same dropout."""
    model.zero_grad(set_to_none=True)
    common.set_seed(seed)
    with common.amp_ctx(amp and batch["input_ids"].is_cuda):
        loss = model(**batch).loss
    loss.backward()
    return {n: p.grad.detach().float().clone() for n, p in model.named_parameters() if p.grad is not None}, float(loss.detach())


def gpu_gib(device: int = 0) -> float:
    """Total memory of the device in GiB (NaN without CUDA)."""
    return torch.cuda.get_device_properties(device).total_memory / 1024 ** 3 if torch.cuda.is_available() else float("nan")
