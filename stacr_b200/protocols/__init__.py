"""Protocol-level building blocks: tensor parallelism, attention-surface compression, checkpoint-boundary
codec, factorisation comparators, planners, profilers and baseline adapters."""
