"""Plain gradient-checkpointing comparator (parity: comparators/checkpointing.py of the reference project)."""

from __future__ import annotations


def enable_gradient_checkpointing(model) -> bool:
    """Turn on block checkpointing through the model's own switch, or by wrapping its transformer blocks."""
    if hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable()
        return True
    try:
        from ..composition import checkpoint_blocks, transformer_blocks

        blocks = transformer_blocks(model)
        checkpoint_blocks(blocks, list(range(len(blocks))))
        return True
    except ValueError:
        return False
