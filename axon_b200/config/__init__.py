"""Typed configurations and the architecture registry."""

from .base import (Architecture, ConfigError, ModelConfig, architecture_of, config_from_dict,
                   known_architectures, load_config, read_config_json, register_architecture,
                   write_config_json)
from .qwen2 import Qwen2Config, qwen2_spec

__all__ = [
    "Architecture", "ConfigError", "ModelConfig", "Qwen2Config", "architecture_of",
    "config_from_dict", "known_architectures", "load_config", "qwen2_spec", "read_config_json",
    "register_architecture", "write_config_json",
]
