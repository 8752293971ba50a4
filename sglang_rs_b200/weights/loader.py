"""Binding of checkpoint tensors to a model, by tensor name.

Storage rule: a bfloat16 tensor is kept in bfloat16, a tensor stored in 32 bits stays
in 32 bits, an integer table becomes int32.  A float16 tensor is kept as it is stored
until a part takes it: the 32-bit path widens it exactly, as the reference does for every
stored float type (``crates/sglang-srt/src/model_artifacts.rs:850-860``), and the bfloat16
path rounds it once.  What a part computes with is the part's business (a matrix is cast
to the compute dtype when the part loads it; a norm's scale is always used in 32-bit).

Tensors that the model does not expect are an error too, except those that match one of
the model's ``ignored_tensors`` patterns: buffers that exporters write and no computation
reads (the reference binds by name and never looks at such entries,
``crates/sglang-srt/src/models/qwen.rs:321-353``).

The whole checkpoint is validated before anything is moved to the device
(reference: ``crates/sglang-srt/src/model_registry.rs:132``,
``crates/sglang-srt/src/model_artifacts.rs:160-191``), and every fault is reported in
one error: missing tensors, unexpected tensors and wrong shapes.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Mapping, Sequence, Tuple

import torch

from .safetensors_io import read_model_dir


class WeightLoadError(ValueError):
    """Lists every missing, unexpected and wrongly shaped tensor at once."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{name} expected {list(want)} found {list(got)}" for name, want, got in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{name} is {dtype}" for name, dtype in self.wrong_dtype))
        super().__init__("\n".join(lines))


def stored_form(tensor: torch.Tensor) -> torch.Tensor:
    """The dtype in which a checkpoint tensor is kept on the host."""
    if tensor.dtype in (torch.bfloat16, torch.float32, torch.int32, torch.float16):
        return tensor
    if tensor.dtype == torch.float64:
        return tensor.to(torch.float32)
    if tensor.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return tensor.to(torch.int32)
    return tensor


def validate(expected: Mapping[str, Tuple[int, ...]], tensors: Mapping[str, torch.Tensor],
             ignored: Sequence[str] = ()) -> None:
    """``ignored``: shell-style patterns of tensor names that may be present and are not read."""
    missing = [name for name in expected if name not in tensors]
    unexpected = [name for name in tensors if name not in expected
                  and not any(fnmatch.fnmatchcase(name, pattern) for pattern in ignored)]
    wrong = [(name, tuple(shape), tuple(tensors[name].shape)) for name, shape in expected.items()
             if name in tensors and tuple(tensors[name].shape) != tuple(shape)]
    wrong_dtype = [(name, str(tensors[name].dtype)) for name in expected
                   if name in tensors and tensors[name].dtype in (torch.complex64, torch.complex128)]
    if missing or unexpected or wrong or wrong_dtype:
        raise WeightLoadError(sorted(missing), sorted(unexpected), sorted(wrong), wrong_dtype)


def load_checkpoint(model_dir: str, expected: Mapping[str, Tuple[int, ...]],
                    ignored: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Reads ``model_dir``, checks it against ``expected`` (name -> shape) and returns the
    tensors in their stored form, on the host."""
    tensors = read_model_dir(model_dir)
    validate(expected, tensors, ignored)
    return {name: stored_form(tensors[name]) for name in expected}
