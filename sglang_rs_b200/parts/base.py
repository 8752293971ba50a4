"""Interfaces of the parts a model is put together from.

A model is a list of blocks; a block arranges a mixer, a feed-forward and norms; a mixer
may use a position encoding.  Each part is constructed from its sizes, its constants and
the checkpoint names of its tensors, and is chosen layer by layer by the architecture's
builder.  No part knows which model it is in.

What each kind must offer:

* every part: ``tensor_specs()`` (checkpoint name -> :class:`TensorSpec`) and
  ``load(tensors, device, dtype)``;
* :class:`Norm`: ``add_norm(residual, delta, out_dtype, row_index=None)``;
* :class:`PositionEncoding`: ``fused_rotary()``: what the fused q/k kernel rotates with: a
  frequency table, or a function from the step's positions to the angle of every (row, pair),
  which covers any encoding of the rotary family; None leaves q and k alone;
* :class:`Mixer`: ``cache_need()`` and ``forward(ctx, cache, x) -> y``;
* :class:`FeedForward`: ``forward(ctx, x) -> y``;
* a block: ``forward(ctx, cache, residual, delta) -> (residual, delta)`` where the hidden
  state is ``residual + delta`` (the sum is taken, in 32-bit, by the next norm).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping, Optional, Tuple, Union

import torch


@dataclass(frozen=True)
class TensorSpec:
    """Shape of a checkpoint tensor and how the random-weights mode fills it:
    ``normal`` N(0, 0.02), ``scale`` 1 + U(-0.1, 0.1), ``zeros``."""
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class PagedKV:
    """A mixer that keeps keys and values per token.  ``window`` None keeps all of them;
    a number keeps only what the last ``window`` positions can still see."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class RequestState:
    """A mixer that keeps a fixed-size state per request (shape without the slot axis).
    ``dtype`` None means the compute dtype."""
    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None


CacheNeed = Union[PagedKV, RequestState, None]


class Part:
    #: True if ``forward`` only launches kernels that read the step's device arrays: nothing is
    #: decided on the host from the step's values, so the call may be captured in a CUDA graph
    graph_safe = False

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        pass


class Norm(Part):
    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    #: True if the fused q/k kernel can apply it from ``fused_rotary()``
    fused = False

    def fused_rotary(self):
        raise NotImplementedError

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed:
        return None

    def split_scratch(self) -> Tuple[int, int]:
        """Floats of scratch per (row, key split) that a split attention run needs:
        (partial accumulators, partial maxima and sums); (0, 0) for mixers without."""
        return (0, 0)

    def forward(self, ctx, cache, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


def matrix_to(tensor: torch.Tensor, device, dtype: torch.dtype) -> torch.Tensor:
    """A projection matrix in the compute dtype on the device (round to nearest even)."""
    return tensor.to(device=device, dtype=dtype).contiguous()


def scale_to(tensor: torch.Tensor, device) -> torch.Tensor:
    """A norm's scale or a bias: always used in 32-bit."""
    return tensor.to(device=device, dtype=torch.float32).contiguous()
