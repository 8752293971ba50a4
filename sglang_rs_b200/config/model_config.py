"""Typed model configuration read from a checkpoint's ``config.json``.

The raw document is kept next to the typed fields so that an architecture's
builder can read any further key it owns.  Nothing here knows a model size: every
number comes from the document.

Behaviour follows the reference's two-stage parse: an all-optional document
(``crates/sglang-srt/src/model_artifacts.rs:387-484``, nested ``text_config``
preferred when it is an object, ``:456-459``) that an architecture adapter turns
into validated fields (``crates/sglang-srt/src/models/qwen.rs:104-244``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Mapping, Sequence


class ConfigError(ValueError):
    """A ``config.json`` that cannot describe a runnable model."""

    def __init__(self, architecture: str, message: str):
        self.architecture = architecture
        super().__init__(f"{architecture}: {message}")


def missing_field(architecture: str, key: str) -> ConfigError:
    return ConfigError(architecture, f"missing required field `{key}`")


@dataclass(frozen=True)
class RawConfig:
    """``config.json`` as a document plus the keys every architecture shares."""

    document: Mapping[str, Any]
    architectures: Sequence[str]
    model_type: str | None
    eos_token_ids: Sequence[int]

    @property
    def text(self) -> Mapping[str, Any]:
        """The sub-document that holds the language model's sizes."""
        nested = self.document.get("text_config")
        return nested if isinstance(nested, dict) else self.document

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "RawConfig":
        if not isinstance(document, dict):
            raise ConfigError("config.json", "top level must be a JSON object")
        architectures = document.get("architectures") or []
        if not isinstance(architectures, list) or not all(isinstance(a, str) for a in architectures):
            raise ConfigError("config.json", "`architectures` must be a list of strings")
        eos = document.get("eos_token_id")
        if eos is None:
            eos_ids: list[int] = []
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = [eos]
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = list(eos)
        else:
            raise ConfigError("config.json", "`eos_token_id` must be an integer or a list of integers")
        model_type = document.get("model_type")
        return cls(document, tuple(architectures), model_type if isinstance(model_type, str) else None, tuple(eos_ids))

    @classmethod
    def from_json(cls, path: str | os.PathLike) -> "RawConfig":
        path = os.fspath(path)
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path, "r", encoding="utf-8") as handle:
                document = json.load(handle)
        except FileNotFoundError:
            raise ConfigError("config.json", f"no such file: {path}") from None
        except json.JSONDecodeError as error:
            raise ConfigError("config.json", f"{path}: invalid JSON: {error}") from None
        return cls.from_dict(document)


def required_positive_int(architecture: str, document: Mapping[str, Any], key: str) -> int:
    """A size that must be present and non-zero (``models/mod.rs:1252-1265``)."""
    value = document.get(key)
    if value is None:
        raise missing_field(architecture, key)
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(architecture, f"`{key}` must be an integer, found {value!r}")
    if value <= 0:
        raise ConfigError(architecture, f"`{key}` must be non-zero")
    return value


def optional_positive_int(architecture: str, document: Mapping[str, Any], key: str) -> int | None:
    if document.get(key) is None:
        return None
    return required_positive_int(architecture, document, key)


def optional_bool(architecture: str, document: Mapping[str, Any], key: str) -> bool | None:
    value = document.get(key)
    if value is None:
        return None
    if not isinstance(value, bool):
        raise ConfigError(architecture, f"`{key}` must be a boolean, found {value!r}")
    return value


def optional_float(architecture: str, document: Mapping[str, Any], key: str) -> float | None:
    value = document.get(key)
    if value is None:
        return None
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(architecture, f"`{key}` must be a number, found {value!r}")
    return float(value)
