from .spec import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, NoPositionSpec,
                   RMSNormSpec, RotarySpec, ScheduleEntry, SwiGLUSpec, default_schedule)
from .qwen3 import ConfigError, Qwen3Config

__all__ = ["AttentionSpec", "EmbeddingSpec", "HeadSpec", "LayerSpec", "ModelSpec", "NoPositionSpec",
           "RMSNormSpec", "RotarySpec", "ScheduleEntry", "SwiGLUSpec", "default_schedule",
           "ConfigError", "Qwen3Config"]
