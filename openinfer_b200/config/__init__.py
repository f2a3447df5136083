"""Typed configurations and the architecture registry."""
from .base import (
    ArchitectureEntry,
    ConfigError,
    ModelConfig,
    known_architectures,
    load_config,
    read_config_json,
    register_architecture,
    resolve_architecture,
    unregister_architecture,
)
from .qwen3 import Qwen3Config

__all__ = [
    "ArchitectureEntry", "ConfigError", "ModelConfig", "Qwen3Config", "known_architectures",
    "load_config", "read_config_json", "register_architecture", "resolve_architecture",
    "unregister_architecture",
]
