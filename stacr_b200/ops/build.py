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


STAMP = HERE / "libstacr_b200.so.stamp"


def source_digest() -> str:
    """Hash of every source and header the library is built from (file times do not survive every copy of a tree)."""
    import hashlib

    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def is_stale() -> bool:
    if not LIB.exists() or not STAMP.exists():
        return True
    return STAMP.read_text().strip() != source_digest()


def build(verbose: bool = False) -> Path:
    """Compile every source and link the library; safe to call from several processes at once.

    Objects go to a directory private to the calling process and the link writes a temporary name that is moved over
    the library with ``os.replace``, so another process either maps the old complete file or the new complete file.
    """
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernel library")
    digest = source_digest()
    (HERE / "build").mkdir(exist_ok=True)
    objdir = HERE / "build" / f"obj.{os.getpid()}"
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
    staged = LIB.with_name(f".{LIB.name}.{os.getpid()}.tmp")
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(staged), *map(str, objs)]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        staged.unlink(missing_ok=True)
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(staged, LIB)
    STAMP.write_text(digest)
    (HERE / "build" / "ptxas.log").write_text("\n".join(f"== {n}\n{log}" for n, log in logs))
    shutil.rmtree(objdir, ignore_errors=True)
    if verbose:
        for name, log in logs:
            print(f"== {name}\n{log}")
    return LIB


def ensure_built() -> Path | None:
    """Build when stale and a compiler is present; return the library path if it exists.

    Processes that arrive together (the ranks of one launcher) serialise on a file lock: the first one builds, the
    others find a fresh library when they get the lock and return without compiling.
    """
    if not is_stale() or nvcc_path() is None:
        return LIB if LIB.exists() else None
    import fcntl

    (HERE / "build").mkdir(exist_ok=True)
    with open(HERE / "build" / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if is_stale():
                build()
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB if LIB.exists() else None


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv)
    print(path)
