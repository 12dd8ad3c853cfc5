"""``stacr``: import-compatible front door of the framework.

Users of the reference package keep ``import stacr``, ``from stacr.surgery import apply_stacr``,
``from stacr.adaptive import STACRConfig`` and ``python -m stacr ...``; every name resolves to the
implementation in ``stacr_b200``.
"""

import importlib
import sys

import stacr_b200 as _impl
from stacr_b200 import *  # noqa: F401,F403
from stacr_b200 import __all__, __version__  # noqa: F401

_SUBMODULES = (
    "adaptive", "adaptive_checkpointing", "analysis", "cli", "composition", "compressor", "datasets", "diagnostics", "hooks",
    "index_compression", "layers", "memory", "memory_accounting", "metrics", "models", "oja", "planner", "quant",
    "rank_controller", "residual", "surgery", "training", "utils", "protocols", "optim", "ops", "parallel", "comparators",
)


def __getattr__(name):
    if name in _SUBMODULES:
        module = importlib.import_module(f"stacr_b200.{name}")
        sys.modules[f"{__name__}.{name}"] = module
        return module
    raise AttributeError(f"module 'stacr' has no attribute {name!r}")


class _AliasFinder:
    """Resolve ``stacr.x.y`` imports to ``stacr_b200.x.y`` modules (same objects, not copies)."""

    @staticmethod
    def find_spec(fullname, path=None, target=None):
        if not fullname.startswith("stacr."):
            return None
        real = "stacr_b200." + fullname[len("stacr."):]
        try:
            module = importlib.import_module(real)
        except ModuleNotFoundError:
            return None
        from importlib.machinery import ModuleSpec

        own = (module.__spec__, getattr(module, "__loader__", None))

        class _Loader:
            @staticmethod
            def create_module(spec):
                return module

            @staticmethod
            def exec_module(mod):
                mod.__spec__, mod.__loader__ = own      # the import system stamped the alias spec on it; put the real one back

        return ModuleSpec(fullname, _Loader(), is_package=hasattr(module, "__path__"))


if not any(isinstance(f, type) and f.__name__ == "_AliasFinder" for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder)
