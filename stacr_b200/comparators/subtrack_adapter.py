"""SubTrack-style optimizer factory (parity: comparators/subtrack_adapter.py:146-224 of the reference project).

The reference loads an external SubTrack++ source tree; here the in-tree ``SubTrackAdamW`` (projected Adam moments with
a Grassmannian-tracked subspace) is built from the same trainer keys.
"""

from __future__ import annotations


import importlib.util
import os
import subprocess
import sys
from pathlib import Path

SUBTRACK_URL = "https://github.com/criticalml-uw/SubTrack"
SUBTRACK_COMMIT = "aabebe310e95a709454d32ce4c697d09114edac9"
SUBTRACK_SOURCE_ENV = "STACR_SUBTRACK_SOURCE"
IN_TREE_REVISION = "in-tree"
INSTALL_COMMAND = (
    f"git clone {SUBTRACK_URL}.git third_party/SubTrack && git -C third_party/SubTrack checkout {SUBTRACK_COMMIT}; "
    f"then set {SUBTRACK_SOURCE_ENV} to that directory"
)


def activate_subtrack_source():
    """Put an upstream SubTrack checkout named by ``STACR_SUBTRACK_SOURCE`` on the import path.

    Returns the checkout's path, or ``None`` when the variable is unset (the in-tree optimizer is used then).
    Raises when the directory lacks the upstream package or another ``low_rank_torch`` is already imported.
    """
    value = os.environ.get(SUBTRACK_SOURCE_ENV)
    if not value:
        return None
    root = Path(value).expanduser().resolve()
    needed = (root / "low_rank_torch" / "__init__.py", root / "utils" / "file_utils.py")
    if not all(f.is_file() for f in needed):
        raise RuntimeError(f"{SUBTRACK_SOURCE_ENV}={root} is not a complete SubTrack checkout")
    loaded = sys.modules.get("low_rank_torch")
    loaded_file = getattr(loaded, "__file__", None)
    if loaded_file and root not in Path(loaded_file).resolve().parents:
        raise RuntimeError("another low_rank_torch package is already imported; start a fresh process")
    if str(root) not in sys.path:
        sys.path.insert(0, str(root))
    return root


def upstream_available() -> bool:
    """True when the upstream ``low_rank_torch`` package can be imported."""
    activate_subtrack_source()
    return importlib.util.find_spec("low_rank_torch") is not None


def subtrack_available() -> bool:
    """Always true: without an upstream checkout the in-tree ``SubTrackAdamW`` serves."""
    activate_subtrack_source()
    return True


def require_subtrack() -> None:
    if not subtrack_available():          # kept for callers that guard on it; cannot fail with the in-tree optimizer
        raise RuntimeError(f"SubTrack is optional; install it with: {INSTALL_COMMAND}")


def _git(root: Path, *args) -> subprocess.CompletedProcess:
    return subprocess.run(["git", "-c", f"safe.directory={root.as_posix()}", "-C", str(root), *args],
                          capture_output=True, text=True, check=False)


def subtrack_revision():
    """Commit of the upstream checkout in use, ``"in-tree"`` for the in-tree optimizer, ``None`` if unknown."""
    root = activate_subtrack_source()
    if root is None:
        return IN_TREE_REVISION
    out = _git(root, "rev-parse", "HEAD")
    return out.stdout.strip() if out.returncode == 0 and out.stdout.strip() else None


def require_pinned_subtrack() -> None:
    """With an upstream checkout selected, insist on the pinned commit and a clean optimizer tree."""
    require_subtrack()
    root = activate_subtrack_source()
    if root is None:
        return
    actual = subtrack_revision()
    if actual != SUBTRACK_COMMIT:
        raise RuntimeError(f"SubTrack comparison needs revision {SUBTRACK_COMMIT}, found {actual or 'unverified'}. {INSTALL_COMMAND}")
    if _git(root, "diff", "HEAD", "--quiet", "--", "low_rank_torch", "utils").returncode:
        raise RuntimeError("the SubTrack checkout has local changes under low_rank_torch/ or utils/")


def create_subtrack_optimizer(model, config):
    from .lowrank_optim import SubTrackAdamW, split_param_groups

    groups = split_param_groups(
        model, config.get("subtrack_target_modules"), float(config.get("weight_decay", 0.0)),
        rank=int(config.get("subtrack_rank", 8)), update_proj_gap=int(config.get("subtrack_update_interval", 200)),
        scale=float(config.get("subtrack_scale", 0.25)), proj_type=config.get("subtrack_proj_type", "std"),
        step_size=float(config.get("subtrack_step_size", 0.1)), track_interval=max(1, int(config.get("subtrack_update_interval", 200)) // 20),
    )
    return SubTrackAdamW(groups, lr=float(config.get("lr", 5e-5)))
