"""Re-exports of the saved-tensor-hook path (parity: stacr/hooks.py of the reference project)."""

from .compressor import PackedActivation, STACRCompressor, STACRConfig, stacr_saved_tensors

__all__ = ["PackedActivation", "STACRCompressor", "STACRConfig", "stacr_saved_tensors"]
