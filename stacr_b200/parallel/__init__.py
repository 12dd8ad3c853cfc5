"""Multi-GPU plumbing: data-parallel gradient sync, tensor-parallel layers, symmetric peer memory."""

from .ddp import GradSync, all_reduce_mean_, broadcast_parameters, init_distributed
from .zero import ShardedGradSync
from .health import CheckpointCorrupt, Heartbeat, RankFailure, guarded, load_checkpoint, verify_checkpoint, write_checkpoint

__all__ = ["GradSync", "ShardedGradSync", "all_reduce_mean_", "broadcast_parameters", "init_distributed", "Heartbeat", "RankFailure", "CheckpointCorrupt", "guarded",
           "write_checkpoint", "verify_checkpoint", "load_checkpoint"]
