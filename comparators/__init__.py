"""``comparators``: import-compatible name of ``stacr_b200.comparators``.

Scripts written against the reference import ``comparators.prac``, ``comparators.galore_adapter`` and so on
(reference: comparators/*.py); every such name resolves to the module of the same name under
``stacr_b200.comparators`` (the same module object, not a copy).
"""

import importlib
import sys
from importlib.machinery import ModuleSpec

import stacr_b200.comparators as _impl
from stacr_b200.comparators import *  # noqa: F401,F403

__path__ = list(_impl.__path__)


class _ComparatorAlias:
    @staticmethod
    def find_spec(fullname, path=None, target=None):
        if not fullname.startswith("comparators."):
            return None
        try:
            module = importlib.import_module("stacr_b200." + fullname)
        except ModuleNotFoundError:
            return None

        own = (module.__spec__, getattr(module, "__loader__", None))

        class _Loader:
            @staticmethod
            def create_module(spec):
                return module

            @staticmethod
            def exec_module(mod):
                mod.__spec__, mod.__loader__ = own      # the import system stamped the alias spec on it; put the real one back

        return ModuleSpec(fullname, _Loader(), is_package=hasattr(module, "__path__"))


if not any(getattr(f, "__name__", "") == "_ComparatorAlias" for f in sys.meta_path):
    sys.meta_path.insert(0, _ComparatorAlias)
