"""Random weights from a configuration and a seed.

Matrices, embeddings and biases are N(0, 0.02); norm scales are 1 + U(-0.1, 0.1).  Each
tensor has its own generator, keyed by the seed and the tensor's name, so a tensor's
values do not depend on which other tensors exist.  Values drawn on the host and values
drawn on a GPU differ (different generators); a model folder written by
:func:`write_model_folder` is the way to give two programs the same weights.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Any, Dict, Mapping

import torch

from ..parts.base import TensorSpec
from .safetensors_io import write_file

NORMAL_STD = 0.02
SCALE_SPREAD = 0.1


def random_tensor(name: str, spec: TensorSpec, seed: int, device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    generator = torch.Generator(device=device)
    generator.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1))
    if spec.init == "normal":
        values = torch.randn(spec.shape, generator=generator, device=device, dtype=torch.float32) * NORMAL_STD
    elif spec.init == "scale":
        values = 1.0 + (torch.rand(spec.shape, generator=generator, device=device, dtype=torch.float32) * 2 - 1) * SCALE_SPREAD
    elif spec.init == "zeros":
        values = torch.zeros(spec.shape, device=device, dtype=torch.float32)
    else:
        raise ValueError(f"tensor {name}: unknown init {spec.init}")
    return values.to(dtype)


def random_tensors(specs: Mapping[str, TensorSpec], seed: int, device="cpu",
                   dtype: torch.dtype = torch.float32) -> Dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, device, dtype) for name, spec in specs.items()}


def write_model_folder(path: str, config_document: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` for the architecture that
    ``config_document`` names, with weights drawn from ``seed`` and stored as ``dtype``."""
    from ..config import RawConfig, resolve_architecture
    from .. import models  # noqa: F401  (registers the architectures)
    raw = RawConfig.from_dict(dict(config_document))
    entry = resolve_architecture(raw)
    model = entry.build_model(entry.parse_config(raw))
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(dict(config_document), handle, indent=1)
    tensors = random_tensors(model.tensor_specs(), seed, "cpu", dtype)
    write_file(os.path.join(path, "model.safetensors"), tensors, {"format": "pt", "seed": str(seed)})
    return path
