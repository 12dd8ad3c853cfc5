"""Build the sm_100a kernel library in-tree with nvcc.

The kernels are plain CUDA C++ with a C ABI (no framework headers), so each file compiles
in seconds and the resulting ``libstacr_b200.so`` is loaded with ctypes.  ``python -m
stacr_b200.ops.build`` rebuilds; ``ensure_built()`` rebuilds only when a source is newer
than the library.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libstacr_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def nvcc_path() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def is_stale() -> bool:
    if not LIB.exists():
        return True
    stamp = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return any(p.stat().st_mtime > stamp for p in deps)


def build(verbose: bool = False) -> Path:
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)
    logs = []

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        logs.append((src.name, proc.stderr))
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources()))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    (objdir / "ptxas.log").write_text("\n".join(f"== {n}\n{log}" for n, log in logs))
    if verbose:
        for name, log in logs:
            print(f"== {name}\n{log}")
    return LIB


def ensure_built() -> Path | None:
    """Build when stale and a compiler is present; return the library path if it exists."""
    if is_stale() and nvcc_path() is not None:
        build()
    return LIB if LIB.exists() else None


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv)
    print(path)
