"""Typed model configuration and the architecture registry."""
from .specs import (ChannelDeltaSpec, ConfigError, EmbeddingSpec, GqaAttentionSpec, LatentAttentionSpec, LayerSpec, LmHeadSpec,
                    ModelConfig, NoPositionSpec, RmsNormSpec, RopeSpec, RunSpec, ScaledEmbeddingSpec, ScaledLmHeadSpec,
                    SquaredReluSpec, SwiGluSpec, UnitOffsetRmsNormSpec)
from .registry import (Architecture, architecture_names, get_architecture, load_config, parse_config,
                       register_architecture)

__all__ = [
    "ConfigError", "EmbeddingSpec", "LmHeadSpec", "GqaAttentionSpec", "LayerSpec", "ModelConfig", "NoPositionSpec", "RmsNormSpec", "RopeSpec",
    "RunSpec", "SwiGluSpec", "ChannelDeltaSpec", "LatentAttentionSpec", "ScaledEmbeddingSpec", "ScaledLmHeadSpec",
    "SquaredReluSpec", "UnitOffsetRmsNormSpec", "Architecture", "architecture_names", "get_architecture", "load_config",
    "parse_config", "register_architecture",
]
