from .spec import (AttentionSpec, DecayStateSpec, EmbeddingSpec, GatedAttentionSpec, HeadSpec, LayerSpec,
                   MatrixMemorySpec, ModelSpec, NoPositionSpec, PairRotarySpec, RMSNormSpec, RotarySpec,
                   ScheduleEntry, SwiGLUSpec, default_schedule)
from .qwen3 import ConfigError, Qwen3Config
from .pugalix import PugalixConfig

__all__ = ["AttentionSpec", "DecayStateSpec", "EmbeddingSpec", "GatedAttentionSpec", "HeadSpec", "LayerSpec",
           "MatrixMemorySpec", "ModelSpec", "NoPositionSpec", "PairRotarySpec", "RMSNormSpec", "RotarySpec",
           "ScheduleEntry", "SwiGLUSpec", "default_schedule", "ConfigError", "Qwen3Config", "PugalixConfig"]
