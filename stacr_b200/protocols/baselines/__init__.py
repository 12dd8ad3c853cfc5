"""Memory baselines that protocols compose with compression: AMP, checkpointing modes, saved-tensor offload,
8-bit optimizer factory and graceful-skip adapters around optional third-party libraries."""
