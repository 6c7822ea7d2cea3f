from .model_config import (ConfigError, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, LayerSpec, MixerSpec,
                           ModelConfig, NormSpec, PositionSpec, RopeScaling)
from .presets import preset, preset_names
from .registry import (architecture, config_from_dict, load_config, part, register_architecture,
                       register_part, registered_architectures)

__all__ = ["ConfigError", "EmbeddingSpec", "FeedForwardSpec", "HeadSpec", "LayerRun", "LayerSpec", "MixerSpec", "ModelConfig",
           "NormSpec", "PositionSpec", "RopeScaling", "architecture", "config_from_dict",
           "load_config", "part", "preset", "preset_names", "register_architecture", "register_part",
           "registered_architectures"]
