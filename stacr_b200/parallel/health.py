"""Host-side failure detection for multi-rank runs.

Nothing here touches a device.  Three pieces:

* :class:`Heartbeat` — every rank writes ``(step, wall time)`` to the job's key-value store between steps and reads
  its peers' entries before it launches the next step.  A rank that stopped (exception, exit, stall) is seen as a
  stale or ``left`` entry, and the survivors raise :class:`RankFailure` *before* they enqueue a collective or an
  in-kernel peer wait that could never complete.
* :func:`guarded` — run a collective with a short process-group timeout and turn the backend's timeout error into
  :class:`RankFailure`; for the cases a heartbeat cannot see (a rank that hangs inside the step).
* :func:`write_checkpoint` / :func:`verify_checkpoint` — checkpoint files carry a SHA-256 sidecar so that a truncated
  or corrupted file is refused at resume instead of half-loaded.

The reference project has no elastic layer at all (its only guards are the non-finite-loss stop and per-cell OOM
capture, stacr/training.py:452-453 and experiments/benchmarks/distributed_data.py:183-191 there); this module is the
detection half of one.  Recovery is restart-from-checkpoint: the survivors exit non-zero and the launcher restarts
the job, which resumes through ``resume_from``.
"""

from __future__ import annotations

import hashlib
import json
import os
import time
from contextlib import contextmanager
from dataclasses import dataclass
from datetime import timedelta
from pathlib import Path
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class RankFailure(RuntimeError):
    """One or more peers stopped making progress.  ``ranks`` lists them; ``reason`` maps rank -> why."""

    def __init__(self, reason: Dict[int, str]):
        self.reason = dict(reason)
        self.ranks = sorted(self.reason)
        super().__init__("rank failure: " + ", ".join(f"rank {r}: {why}" for r, why in sorted(self.reason.items())))


class CheckpointCorrupt(RuntimeError):
    pass


@dataclass
class Beat:
    step: int
    time: float
    state: str = "alive"   # alive | left | failed

    def dump(self) -> bytes:
        return json.dumps({"step": self.step, "time": self.time, "state": self.state}).encode()

    @classmethod
    def load(cls, raw: bytes) -> "Beat":
        d = json.loads(bytes(raw).decode())
        return cls(int(d["step"]), float(d["time"]), d.get("state", "alive"))


class Heartbeat:
    """Per-rank liveness entries in a ``torch.distributed`` store (TCPStore, FileStore, or the default group's store).

    ``beat(step)`` is called once per step, after the step's device work has been enqueued and before the next one;
    ``check()`` raises :class:`RankFailure` when a peer is ``failed``/``left``, more than ``max_lag`` steps behind, or
    silent for more than ``timeout`` seconds.  ``leave()`` marks an orderly exit between steps; ``fail(msg)`` is
    called from an exception handler so that peers stop at their next check instead of waiting for a timeout.
    """

    def __init__(self, store, rank: int, world: int, *, timeout: float = 30.0, max_lag: Optional[int] = None, prefix: str = "hb"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout, self.max_lag, self.prefix = float(timeout), max_lag, prefix
        self.step = -1
        self._put(Beat(-1, time.time()))

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def _put(self, beat: Beat) -> None:
        self.store.set(self._key(self.rank), beat.dump())

    def beat(self, step: int) -> None:
        self.step = int(step)
        self._put(Beat(self.step, time.time()))

    def leave(self) -> None:
        self._put(Beat(self.step, time.time(), "left"))

    def fail(self, message: str = "") -> None:
        self._put(Beat(self.step, time.time(), "failed" + (f": {message[:200]}" if message else "")))

    def peers(self) -> Dict[int, Optional[Beat]]:
        out: Dict[int, Optional[Beat]] = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            key = self._key(r)
            try:
                present = self.store.check([key])
            except Exception:  # noqa: BLE001 - store flavours without check(): fall through to get with the store's own timeout
                present = True
            out[r] = Beat.load(self.store.get(key)) if present else None
        return out

    def check(self, now: Optional[float] = None) -> None:
        now = time.time() if now is None else now
        bad: Dict[int, str] = {}
        for r, beat in self.peers().items():
            if beat is None:
                bad[r] = "never registered"
            elif beat.state != "alive":
                bad[r] = f"{beat.state} at step {beat.step}"
            elif now - beat.time > self.timeout:
                bad[r] = f"silent for {now - beat.time:.1f}s (last step {beat.step})"
            elif self.max_lag is not None and self.step - beat.step > self.max_lag:
                bad[r] = f"{self.step - beat.step} steps behind"
        if bad:
            raise RankFailure(bad)

    @contextmanager
    def guard(self):
        """Publish ``failed`` when the body raises, so peers learn of it at their next ``check()``."""
        try:
            yield self
        except BaseException as exc:
            self.fail(f"{type(exc).__name__}: {exc}")
            raise


_TIMEOUT_MARKERS = ("timed out", "timeout", "Connection closed by peer", "Connection reset by peer", "Broken pipe")


def guarded(fn, *args, what: str = "collective", **kwargs):
    """Call a collective and convert a backend timeout or a broken connection into :class:`RankFailure`."""
    try:
        return fn(*args, **kwargs)
    except RuntimeError as exc:  # DistBackendError derives from RuntimeError
        text = str(exc)
        if any(m.lower() in text.lower() for m in _TIMEOUT_MARKERS):
            raise RankFailure({-1: f"{what} did not complete: {text.splitlines()[0][:200]}"}) from exc
        raise


def short_timeout_group(seconds: float, backend: Optional[str] = None):
    """A process group over all ranks whose collectives give up after ``seconds`` (for the step-boundary health check)."""
    return dist.new_group(backend=backend, timeout=timedelta(seconds=seconds))


# ------------------------------------------------------------------------------------------------ checkpoint integrity
def _digest(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def write_checkpoint(obj, path) -> Path:
    """``torch.save`` to a temporary name, fsync, rename, then write ``<path>.sha256`` (size and digest)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(path.name + ".tmp")
    with tmp.open("wb") as fh:
        torch.save(obj, fh)
        fh.flush()
        os.fsync(fh.fileno())
    os.replace(tmp, path)
    path.with_name(path.name + ".sha256").write_text(json.dumps({"bytes": path.stat().st_size, "sha256": _digest(path)}), encoding="utf-8")
    return path


def verify_checkpoint(path, *, require_sidecar: bool = False) -> bool:
    """Raise :class:`CheckpointCorrupt` if the file does not match its sidecar; ``False`` when there is no sidecar."""
    path = Path(path)
    if not path.is_file():
        raise CheckpointCorrupt(f"{path}: missing")
    side = path.with_name(path.name + ".sha256")
    if not side.is_file():
        if require_sidecar:
            raise CheckpointCorrupt(f"{path}: no integrity record")
        return False
    want = json.loads(side.read_text(encoding="utf-8"))
    size = path.stat().st_size
    if size != int(want["bytes"]):
        raise CheckpointCorrupt(f"{path}: {size} bytes on disk, {want['bytes']} recorded (truncated write?)")
    if _digest(path) != want["sha256"]:
        raise CheckpointCorrupt(f"{path}: content digest mismatch")
    return True


def load_checkpoint(path, *, map_location="cpu", require_sidecar: bool = False):
    verify_checkpoint(path, require_sidecar=require_sidecar)
    return torch.load(path, map_location=map_location, weights_only=False)


def latest_valid_checkpoint(paths: List) -> Optional[Path]:
    """The newest file (by mtime) that passes verification; corrupt ones are skipped."""
    for p in sorted((Path(x) for x in paths), key=lambda q: q.stat().st_mtime if q.exists() else 0, reverse=True):
        try:
            verify_checkpoint(p)
            return p
        except CheckpointCorrupt:
            continue
    return None
