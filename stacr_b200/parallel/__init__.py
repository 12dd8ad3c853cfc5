"""Multi-GPU plumbing: data-parallel gradient sync, tensor-parallel layers, symmetric peer memory."""

from .ddp import GradSync, all_reduce_mean_, broadcast_parameters, init_distributed

__all__ = ["GradSync", "all_reduce_mean_", "broadcast_parameters", "init_distributed"]
