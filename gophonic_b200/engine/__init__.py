from .model import Model, dtype_mode
from .step import Engine, StepBatch, StepError, build_batch, choose_splits

__all__ = ["Engine", "Model", "StepBatch", "StepError", "build_batch", "choose_splits", "dtype_mode"]
