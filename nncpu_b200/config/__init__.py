"""Configuration: typed per-architecture classes and the specs they produce."""
from .registry import (architectures, config_class, config_from_dict, load_config,
                       register_architecture)
from .specs import (AttentionSpec, BlockSpec, EmbeddingSpec, FeedForwardSpec, GatedMlpSpec,
                    MixerSpec, ModelSpec, NormSpec, OutputSpec, PositionSpec, ScheduleEntry)
from .qwen3 import Qwen3Config

__all__ = [
    "architectures", "config_class", "config_from_dict", "load_config", "register_architecture",
    "AttentionSpec", "BlockSpec", "EmbeddingSpec", "FeedForwardSpec", "GatedMlpSpec", "MixerSpec",
    "ModelSpec", "NormSpec", "OutputSpec", "PositionSpec", "ScheduleEntry", "Qwen3Config",
]
