"""GaLore optimizer factory under the name the protocol package uses (the implementation lives with the comparators).

Parity: stacr/protocols/baselines/galore_adapter.py of the reference project.
"""

from ...comparators.galore_adapter import create_galore_optimizer, galore_available  # noqa: F401

__all__ = ["create_galore_optimizer", "galore_available"]
