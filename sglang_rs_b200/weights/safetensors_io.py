"""Reader and writer for the safetensors container.

Layout (checked as the reference checks it,
``crates/sglang-srt/src/model_artifacts.rs:1456-1514``, ``:1533-1590``): eight bytes of
little-endian header length, a JSON header (``__metadata__`` skipped) that gives
``dtype``, ``shape`` and ``data_offsets`` per tensor, then the payload.  A tensor's
byte length must equal ``prod(shape) * width`` and must lie inside the file.

Shard discovery follows ``model_artifacts.rs:495-515``: ``model.safetensors.index.json``
if it exists (a shard it names must exist), else every ``*.safetensors`` in name order.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, Mapping, Tuple

import numpy as np
import torch

#: safetensors dtype string -> (torch dtype, bytes per element)
DTYPES: Dict[str, Tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def read_header(path: str) -> Tuple[dict, int]:
    """Returns the tensor table and the offset at which the payload starts."""
    size = os.path.getsize(path)
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise SafetensorsError(f"{path}: shorter than the 8-byte header length")
        (header_len,) = struct.unpack("<Q", prefix)
        if header_len > size - 8:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file ({size} bytes)")
        try:
            header = json.loads(handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: header is not valid JSON: {error}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header must be a JSON object")
    header.pop("__metadata__", None)
    payload = size - 8 - header_len
    for name, entry in header.items():
        try:
            dtype, shape, (begin, end) = entry["dtype"], entry["shape"], entry["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: tensor {name}: malformed header entry") from None
        if dtype not in DTYPES:
            raise SafetensorsError(f"{path}: tensor {name}: unsupported dtype {dtype}")
        count = 1
        for extent in shape:
            count *= int(extent)
        if end - begin != count * DTYPES[dtype][1]:
            raise SafetensorsError(
                f"{path}: tensor {name}: {end - begin} bytes do not match shape {shape} of {dtype}")
        if begin < 0 or end > payload:
            raise SafetensorsError(f"{path}: tensor {name}: bytes {begin}..{end} lie outside the payload ({payload})")
    return header, 8 + header_len


def read_file(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of one file, as views of a private copy-on-write mapping."""
    header, base = read_header(path)
    if not header:
        return {}
    mapping = np.memmap(path, dtype=np.uint8, mode="c")
    whole = torch.from_numpy(mapping)
    tensors: Dict[str, torch.Tensor] = {}
    for name, entry in header.items():
        dtype, _ = DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        flat = whole[base + begin: base + end]
        if (base + begin) % DTYPES[entry["dtype"]][1] != 0:
            flat = flat.clone()          # a view must be aligned to its element size
        tensors[name] = flat.view(dtype).reshape([int(extent) for extent in entry["shape"]])
    return tensors


def shard_files(model_dir: str) -> list[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as handle:
            weight_map = json.load(handle).get("weight_map", {})
        names = sorted(set(weight_map.values()))
        for name in names:
            if not os.path.exists(os.path.join(model_dir, name)):
                raise SafetensorsError(f"{index} names shard {name}, which does not exist")
        return [os.path.join(model_dir, name) for name in names]
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"{model_dir}: no *.safetensors file")
    return [os.path.join(model_dir, name) for name in names]


def read_model_dir(model_dir: str) -> Dict[str, torch.Tensor]:
    tensors: Dict[str, torch.Tensor] = {}
    for path in shard_files(model_dir):
        for name, tensor in read_file(path).items():
            tensors.setdefault(name, tensor)   # first shard in order wins, as in the reference
    return tensors


def write_file(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    ordered: Iterable[Tuple[str, torch.Tensor]] = sorted(tensors.items())
    for name, tensor in ordered:
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {tensor.dtype} cannot be stored")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    # written beside the target and moved over it, so that a mapping of the old file stays valid
    partial = f"{path}.{os.getpid()}.tmp"
    with open(partial, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in sorted(tensors.items()):
            data = tensor.detach().contiguous().cpu()
            handle.write(data.reshape(-1).view(torch.uint8).numpy().tobytes() if data.numel() else b"")
    os.replace(partial, path)
