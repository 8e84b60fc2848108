from .base import (AttentionSpec, BlockSpec, ConfigError, GatedFeedForwardSpec, LayerCall,
                   ModelSpec, NormSpec, RotarySpec, default_schedule)
from .registry import (load_config, read_config_json, register_architecture,
                       registered_architectures, resolve_architecture)
from .gemma3 import Gemma3Config

__all__ = [
    "AttentionSpec", "BlockSpec", "ConfigError", "GatedFeedForwardSpec", "LayerCall",
    "ModelSpec", "NormSpec", "RotarySpec", "default_schedule", "load_config",
    "read_config_json", "register_architecture", "registered_architectures",
    "resolve_architecture", "Gemma3Config",
]
