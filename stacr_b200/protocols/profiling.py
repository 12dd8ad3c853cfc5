"""Phase profiler: nested ``step`` / ``phase`` scopes that record time and memory peaks to JSONL.

The JSONL schema (a ``meta`` line followed by one ``step`` line with per-phase records) follows
stacr/protocols/profiling.py:29-491 of the reference project.  Timing differs by design: on CUDA each phase is
bracketed by CUDA events on the current stream and read after one synchronisation at the end of the step,
instead of synchronising at every phase boundary; memory peaks still come from the allocator statistics.
On CPU, resident set size is reported (never silent zeros).
"""

from __future__ import annotations

import json
import os
import platform
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Optional

import torch


def cuda_sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def reset_peaks():
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def _rss() -> int:
    try:
        import psutil

        return int(psutil.Process().memory_info().rss)
    except Exception:
        try:
            with open("/proc/self/statm") as fh:
                return int(fh.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
        except Exception:
            return -1


def read_peaks() -> Dict[str, Any]:
    if torch.cuda.is_available():
        return {"mode": "cuda", "allocated_bytes": torch.cuda.memory_allocated(), "reserved_bytes": torch.cuda.memory_reserved(),
                "peak_allocated_bytes": torch.cuda.max_memory_allocated(), "peak_reserved_bytes": torch.cuda.max_memory_reserved()}
    rss = _rss()
    return {"mode": "cpu", "rss_bytes": rss, "peak_rss_bytes": rss}


def capture_environment() -> Dict[str, Any]:
    env = {"python": platform.python_version(), "platform": platform.platform(), "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
           "cuda_available": torch.cuda.is_available(), "cuda_launch_blocking": os.environ.get("CUDA_LAUNCH_BLOCKING"),
           "alloc_conf": os.environ.get("PYTORCH_CUDA_ALLOC_CONF")}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(0)
        env.update(gpu=p.name, gpu_memory_bytes=p.total_memory, sm_count=p.multi_processor_count, capability=list(torch.cuda.get_device_capability(0)))
    return env


@dataclass
class PhaseResult:
    time_ms: float = 0.0
    start_allocated_bytes: int = 0
    start_reserved_bytes: int = 0
    peak_allocated_bytes: int = 0
    peak_reserved_bytes: int = 0
    end_allocated_bytes: int = 0
    end_reserved_bytes: int = 0
    delta_peak_allocated_bytes: int = 0
    delta_peak_reserved_bytes: int = 0
    start_rss_bytes: int = 0
    peak_rss_bytes: int = 0
    end_rss_bytes: int = 0
    call_count: int = 1


@dataclass
class StepProfile:
    step: int
    device: str
    mode: str
    global_peak_allocated_bytes: int = 0
    global_peak_reserved_bytes: int = 0
    global_peak_rss_bytes: int = 0
    time_ms: float = 0.0
    phases: Dict[str, PhaseResult] = field(default_factory=dict)


_CUDA_ONLY = ("start_allocated_bytes", "start_reserved_bytes", "peak_allocated_bytes", "peak_reserved_bytes", "end_allocated_bytes",
              "end_reserved_bytes", "delta_peak_allocated_bytes", "delta_peak_reserved_bytes")
_CPU_ONLY = ("start_rss_bytes", "peak_rss_bytes", "end_rss_bytes")


class PhaseProfiler:
    def __init__(self, device: str = "auto", out_path: Optional[str] = None, enabled: bool = True):
        cuda = torch.cuda.is_available() and (device == "auto" or str(device).startswith("cuda"))
        self.mode = "cuda" if cuda else "cpu"
        self.device = "cuda" if cuda else "cpu"
        self.out_path, self.enabled = out_path, enabled
        self._current: Optional[StepProfile] = None
        self._last: Optional[StepProfile] = None
        self._pending: list = []  # (phase name, start event, end event) resolved at step end
        self._meta_written = False

    # ------------------------------------------------------------------ metadata
    def write_metadata(self, extra: Optional[Dict[str, Any]] = None) -> None:
        if not self.out_path or self._meta_written:
            return
        os.makedirs(os.path.dirname(os.path.abspath(self.out_path)), exist_ok=True)
        with open(self.out_path, "a") as fh:
            fh.write(json.dumps({"type": "meta", "environment": capture_environment(), **(extra or {})}) + "\n")
        self._meta_written = True

    # ------------------------------------------------------------------ scopes
    @contextmanager
    def step(self, step_idx: int):
        if not self.enabled:
            yield
            return
        self.write_metadata()
        self._current = StepProfile(step=int(step_idx), device=self.device, mode=self.mode)
        self._pending = []
        if self.mode == "cuda":
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            cur = self._current
            if self.mode == "cuda":
                e1.record()
                torch.cuda.synchronize()
                cur.time_ms = e0.elapsed_time(e1)
                for name, a, b in self._pending:
                    cur.phases[name].time_ms += a.elapsed_time(b)
                cur.global_peak_allocated_bytes = torch.cuda.max_memory_allocated()
                cur.global_peak_reserved_bytes = torch.cuda.max_memory_reserved()
            else:
                cur.time_ms = (time.perf_counter() - t0) * 1e3
                cur.global_peak_rss_bytes = max([_rss()] + [p.peak_rss_bytes for p in cur.phases.values()])
            self._write_step()
            self._last, self._current = cur, None

    @contextmanager
    def phase(self, name: str, reset_peaks: bool = True, **extra):
        cur = self._current
        if not self.enabled or cur is None:
            yield
            return
        rec = PhaseResult()
        if self.mode == "cuda":
            if reset_peaks:
                torch.cuda.reset_peak_memory_stats()
            rec.start_allocated_bytes, rec.start_reserved_bytes = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        else:
            rec.start_rss_bytes = _rss()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.mode == "cuda":
                b.record()
                rec.end_allocated_bytes, rec.end_reserved_bytes = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
                rec.peak_allocated_bytes, rec.peak_reserved_bytes = torch.cuda.max_memory_allocated(), torch.cuda.max_memory_reserved()
                rec.delta_peak_allocated_bytes = rec.peak_allocated_bytes - rec.start_allocated_bytes
                rec.delta_peak_reserved_bytes = rec.peak_reserved_bytes - rec.start_reserved_bytes
                rec.time_ms = 0.0
                self._pending.append((name, a, b))
            else:
                rec.end_rss_bytes = _rss()
                rec.peak_rss_bytes = max(rec.start_rss_bytes, rec.end_rss_bytes)
                rec.time_ms = (time.perf_counter() - t0) * 1e3
            seen = cur.phases.get(name)
            if seen is None:
                cur.phases[name] = rec
            else:  # repeated phase: sum time, max peaks
                seen.time_ms += rec.time_ms
                seen.call_count += 1
                for key in ("peak_allocated_bytes", "peak_reserved_bytes", "delta_peak_allocated_bytes", "delta_peak_reserved_bytes", "peak_rss_bytes"):
                    setattr(seen, key, max(getattr(seen, key), getattr(rec, key)))
                seen.end_allocated_bytes, seen.end_reserved_bytes, seen.end_rss_bytes = rec.end_allocated_bytes, rec.end_reserved_bytes, rec.end_rss_bytes

    # ------------------------------------------------------------------ output
    def _write_step(self) -> None:
        cur = self._current
        if not self.out_path or cur is None:
            return
        glob: Dict[str, Any] = {"time_ms": cur.time_ms}
        if cur.mode == "cuda":
            glob.update(peak_allocated_bytes=cur.global_peak_allocated_bytes, peak_reserved_bytes=cur.global_peak_reserved_bytes)
        else:
            glob["peak_rss_bytes"] = cur.global_peak_rss_bytes
        drop = _CPU_ONLY if cur.mode == "cuda" else _CUDA_ONLY
        phases = {name: {k: v for k, v in asdict(p).items() if k not in drop} for name, p in cur.phases.items()}
        with open(self.out_path, "a") as fh:
            fh.write(json.dumps({"type": "step", "step": cur.step, "device": cur.device, "mode": cur.mode, "global": glob, "phases": phases}) + "\n")

    def get_last_step(self) -> Optional[StepProfile]:
        return self._last


@contextmanager
def CudaProfile(section: str):
    """One-shot peak + elapsed report for a code section (printed on exit)."""
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    t0 = time.perf_counter()
    result: Dict[str, Any] = {"section": section}
    try:
        yield result
    finally:
        if cuda:
            b.record()
            torch.cuda.synchronize()
            result.update(time_ms=a.elapsed_time(b), peak_allocated_bytes=torch.cuda.max_memory_allocated())
        else:
            result.update(time_ms=(time.perf_counter() - t0) * 1e3, peak_rss_bytes=_rss())
        print(f"[profile] {section}: {result}")
