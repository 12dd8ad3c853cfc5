from .training import BaselineConfig, OptimizerConfig, TrainingConfig

__all__ = ["BaselineConfig", "OptimizerConfig", "TrainingConfig"]
