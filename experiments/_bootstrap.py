"""Import side effect for scripts run by path (``python experiments/train.py``): put the repository root on ``sys.path``."""

from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
