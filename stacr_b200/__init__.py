"""stacr_b200: Blackwell-native activation-compression training framework (STAC-R capabilities).

Public API mirrors the reference package's ``stacr/__init__.py`` export list.
"""

from .adaptive import AdaptiveSTACRConfig, AdaptiveSTACRLinear, apply_adaptive_stacr, set_stacr_runtime_state
from .compressor import STACRCompressor, STACRConfig, stacr_saved_tensors
from .layers import STACRFunction, STACRLinear
from .memory import saved_surface_predictor, stacr_stored_bytes
from .metrics import cosine_similarity, relative_mse
from .quant import quantize_values
from .surgery import apply_stacr, select_target_names, set_step

__version__ = "0.1.0"

__all__ = [
    "STACRConfig",
    "STACRCompressor",
    "stacr_saved_tensors",
    "STACRFunction",
    "STACRLinear",
    "apply_stacr",
    "select_target_names",
    "set_step",
    "quantize_values",
    "stacr_stored_bytes",
    "saved_surface_predictor",
    "cosine_similarity",
    "relative_mse",
    "AdaptiveSTACRConfig",
    "AdaptiveSTACRLinear",
    "apply_adaptive_stacr",
    "set_stacr_runtime_state",
]
