"""Typed configurations and the architecture registry."""

from .base import ConfigError, ModelConfig
from .qwen3 import Qwen3Config
from .registry import (Architecture, architecture_name, get_architecture, known_architectures, preset_config,
                       read_config, register_architecture)

__all__ = [n for n in dir() if not n.startswith("_")]
