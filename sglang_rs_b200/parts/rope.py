"""Rotary position encoding.

inv_freq[i] = theta^(-2i / rotary_dim), computed in 64-bit and stored in 32-bit
(reference: crates/sglang-kernel/src/rotary.rs:72-98); angle = float(pos) * inv_freq[i];
pairs are (i, i + rotary_dim/2) in the half-split ("NeoX") style or (2i, 2i + 1)
interleaved (rotary.rs:216-236).  Default scaling only, magnitude 1 (rotary.rs:100-103).
The table is a constant of the model; the rotation itself runs inside the fused q/k
kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from .base import PositionEncoding


@dataclass(frozen=True)
class FusedRotary:
    """What the fused q/k kernel needs to rotate: either a table ``inv_freq`` (angle = position *
    inv_freq[i]) or ``angles(positions) -> float32 [rows, rotary_dim / 2]`` for encodings whose angles
    are not a product of position and frequency."""
    inv_freq: Optional[torch.Tensor]
    rotary_dim: int
    interleaved: bool
    angles: Optional[Callable[[torch.Tensor], torch.Tensor]] = None


class RotaryEncoding(PositionEncoding):
    graph_safe = True

    fused = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None, interleaved: bool = False):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        self.theta = float(theta)
        self.interleaved = bool(interleaved)
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rotary_dim} must be even, positive and at most {self.head_dim}")
        if not self.theta > 0:
            raise ValueError("RoPE theta must be finite and positive")
        self._table: Optional[FusedRotary] = None

    def inverse_frequencies(self) -> torch.Tensor:
        pair = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * pair / self.rotary_dim).to(torch.float32)

    def load(self, tensors, device, dtype) -> None:
        # an encoding that several layers share is loaded once: they then share one table on the device
        if self._table is None or self._table.inv_freq.device != torch.device(device):
            self._table = FusedRotary(self.inverse_frequencies().to(device), self.rotary_dim, self.interleaved)

    def fused_rotary(self) -> FusedRotary:
        return self._table


class NoPositionEncoding(PositionEncoding):
    """Leaves q and k as they are."""
    graph_safe = True

    fused = True

    def fused_rotary(self):
        return None
