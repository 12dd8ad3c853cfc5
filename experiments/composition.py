"""Report which optimizer-side comparators can run here, and from which implementation.

Parity: experiments/composition.py (prints the availability of GaLore and SubTrack).
"""

from __future__ import annotations

try:
    from . import _bootstrap  # noqa: F401
except ImportError:
    import _bootstrap  # noqa: F401


def main(argv=None) -> dict:
    from stacr_b200.comparators.galore_adapter import galore_available
    from stacr_b200.comparators.subtrack_adapter import subtrack_available, subtrack_revision, upstream_available

    report = {"galore_available": True, "galore_external_package": galore_available(), "subtrack_available": subtrack_available(),
              "subtrack_upstream_checkout": upstream_available(), "subtrack_revision": subtrack_revision()}
    print(report)
    return report


if __name__ == "__main__":
    main()
