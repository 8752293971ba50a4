from .model_config import (ConfigError, RawConfig, missing_field, optional_bool, optional_float,
                           optional_positive_int, required_positive_int)
from .registry import (ArchitectureEntry, register_architecture, registered_architectures,
                       resolve_architecture, unregister_architecture)

__all__ = [
    "ConfigError", "RawConfig", "ArchitectureEntry", "register_architecture", "registered_architectures",
    "resolve_architecture", "unregister_architecture", "missing_field", "optional_bool", "optional_float",
    "optional_positive_int", "required_positive_int",
]
