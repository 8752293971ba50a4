"""RMSNorm, fused with the residual sum that precedes it.

y = x / sqrt(mean(x^2) + eps) * w with eps inside the root and the weight multiplying
directly (reference: crates/sglang-kernel/src/cpu.rs:26-34).  The sum x = residual + delta,
the mean of squares and the scaling are 32-bit; only the result is rounded to the
compute dtype.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Norm, TensorSpec, scale_to


class RmsNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.width,), "scale")}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.weight = scale_to(tensors[self.weight_name], device)

    def native_record(self):
        """This norm for the step executor: its scale, eps and width."""
        from ..ops.records import SxNorm
        return None if self.weight is None else SxNorm(self.weight.data_ptr(), self.eps, self.width)

    def add_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                 row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        """residual += delta (in place, unless rows are picked); returns norm(residual).
        ``delta`` may be float32 [parts, rows, width]: partial sums, added in order."""
        rows = residual.shape[0] if row_index is None else row_index.numel()
        out = torch.empty((rows, self.width), dtype=out_dtype, device=residual.device)
        ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, row_index=row_index,
                        write_residual=row_index is None)
        return out
