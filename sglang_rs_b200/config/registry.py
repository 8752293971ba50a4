"""One registry from an architecture's name to its configuration and model.

The first entry of ``architectures`` that is registered wins, and the error for an
unknown name lists what is registered, as in the reference
(``crates/sglang-srt/src/model_registry.rs:39-75``, ``:358-390``).

An architecture is added with :func:`register_architecture`; nothing else in the
framework has to change.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .model_config import ConfigError, RawConfig


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    #: RawConfig -> the architecture's typed, validated configuration
    parse_config: Callable[[RawConfig], Any]
    #: typed configuration -> an unloaded model (parts assembled, no weights yet)
    build_model: Callable[[Any], Any]


_REGISTRY: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, parse_config: Callable[[RawConfig], Any],
                          build_model: Callable[[Any], Any], *, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture {name} is already registered")
    _REGISTRY[name] = ArchitectureEntry(name, parse_config, build_model)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_REGISTRY)


def resolve_architecture(raw: RawConfig) -> ArchitectureEntry:
    if not raw.architectures:
        raise ConfigError("config.json", "missing `architectures`; cannot choose a model")
    for name in raw.architectures:
        entry = _REGISTRY.get(name)
        if entry is not None:
            return entry
    raise ConfigError(
        "config.json",
        f"unsupported architectures {list(raw.architectures)}; supported: {registered_architectures()}",
    )
