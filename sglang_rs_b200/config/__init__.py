from .model_config import ConfigError, Qwen3Config, RawConfig
from .registry import (ArchitectureEntry, register_architecture, registered_architectures,
                       resolve_architecture, unregister_architecture)

__all__ = [
    "ConfigError", "Qwen3Config", "RawConfig", "ArchitectureEntry", "register_architecture",
    "registered_architectures", "resolve_architecture", "unregister_architecture",
]
