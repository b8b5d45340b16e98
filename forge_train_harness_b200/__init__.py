"""B200-native pre-training engine and alignment-gate harness.

The public training contract is ``RunConfig`` + ``run_training_loop`` (the counterpart of the reference's
``TrainLoopConfig`` / ``run_training_loop``, workload/src/training_engine_tensor/__init__.py:18-20).
"""
from .config.schema import (CkptConfig, DataConfig, ModelConfig, OptimConfig, ParallelConfig, RunConfig,
                            TrainConfig, preset)
from .engine import Trainer, run_training_loop

__version__ = "0.1.0"
__all__ = ["RunConfig", "ModelConfig", "OptimConfig", "ParallelConfig", "TrainConfig", "DataConfig", "CkptConfig",
           "preset", "Trainer", "run_training_loop"]
