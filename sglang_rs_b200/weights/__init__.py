"""From a model folder (or a configuration and a seed) to a loaded model."""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from .loader import WeightLoadError, load_checkpoint, stored_form, validate
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, read_file, read_model_dir, write_file

__all__ = [
    "WeightLoadError", "load_checkpoint", "stored_form", "validate", "random_tensor", "random_tensors",
    "write_model_folder", "SafetensorsError", "read_file", "read_model_dir", "write_file", "load_model",
    "build_model", "parse_dtype",
]


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.float32, torch.bfloat16):
            return name
    elif name in ("float32", "fp32", "f32"):
        return torch.float32
    elif name in ("bfloat16", "bf16"):
        return torch.bfloat16
    raise ValueError(f"dtype must be bfloat16 or float32, not {name!r}")


def build_model(config_source):
    """An unloaded model from a folder, a config.json path or a config document."""
    from .. import models  # noqa: F401
    from ..config import RawConfig, resolve_architecture
    raw = RawConfig.from_dict(dict(config_source)) if isinstance(config_source, Mapping) \
        else RawConfig.from_json(config_source)
    entry = resolve_architecture(raw)
    config = entry.parse_config(raw)
    return entry.build_model(config), config


def load_model(model_path: Optional[str] = None, *, device="cuda", dtype="bfloat16",
               random_weights: bool = False, seed: int = 0, config: Optional[Mapping[str, Any]] = None):
    """The model that ``config.json`` names, with weights from the folder's safetensors, or,
    with ``random_weights``, drawn from ``seed`` directly on the device (the folder then
    needs only its config.json; ``config`` may stand in for the folder)."""
    dtype = parse_dtype(dtype)
    model, typed = build_model(config if config is not None else model_path)
    specs = model.tensor_specs()
    if random_weights:
        tensors = {}
        for name, spec in specs.items():
            tensors[name] = random_tensor(name, spec, seed, device, dtype if spec.init == "normal" else torch.float32)
    else:
        if model_path is None:
            raise ValueError("a model folder is needed unless random_weights is set")
        tensors = load_checkpoint(model_path, {name: spec.shape for name, spec in specs.items()},
                                  tuple(getattr(model, "ignored_tensors", ())))
    model.load(tensors, device, dtype)
    model.config = typed
    return model
