from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .llama import LlamaConfig, RopeScaling, parse_rope_scaling
from .registry import (Architecture, known_architectures, parse_config, register_architecture,
                       resolve_architecture)

__all__ = ["ConfigError", "LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "LlamaConfig",
           "RopeScaling", "parse_rope_scaling", "Architecture", "known_architectures", "parse_config",
           "register_architecture", "resolve_architecture"]
