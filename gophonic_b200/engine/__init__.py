from .model import Model, dtype_mode
from .step import Engine, StepBatch, StepError, build_batch

__all__ = ["Engine", "Model", "StepBatch", "StepError", "build_batch", "dtype_mode"]
