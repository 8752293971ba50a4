"""Gated feed-forward: down( act(gate(x)) * up(x) ).

With SiLU, act_j = g_j / (1 + exp(-g_j)) * u_j (reference: crates/sglang-kernel/src/cpu.rs:119-123;
order of products crates/sglang-srt/src/cpu_reference.rs:585-603).  gate and up come from
one product with the two matrices stacked (gate rows first), made at load time.  The
activation is a name that the kernels know (``ops.ACTIVATIONS``); it travels to the epilogue of
the gate/up product as a number, so another activation is a case in csrc/activations.cuh and
a name there, not a change to a product kernel.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Mapping

import torch

from .. import ops
from .base import FeedForward, TensorSpec, matrix_to


@dataclass(frozen=True)
class GatedMlpNames:
    gate: str
    up: str
    down: str


class GatedMlp(FeedForward):
    graph_safe = True

    def __init__(self, hidden: int, inner: int, activation: str, names: GatedMlpNames):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unsupported activation {activation}; available: {sorted(ops.ACTIVATIONS)}")
        self.hidden, self.inner, self.activation, self.names = int(hidden), int(inner), activation, names
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        n = self.names
        return {n.gate: TensorSpec((self.inner, self.hidden)), n.up: TensorSpec((self.inner, self.hidden)),
                n.down: TensorSpec((self.hidden, self.inner))}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        n = self.names
        self.w_gate_up = matrix_to(torch.cat([tensors[n.gate], tensors[n.up]], dim=0), device, dtype)
        self.w_down = matrix_to(tensors[n.down], device, dtype)

    def native_record(self):
        """This feed-forward for the step executor: the two stacked matrices, the inner width, the activation."""
        from ..ops.records import SxGatedMlp, linear_record
        if self.w_gate_up is None:
            return None
        return SxGatedMlp(linear_record(self.w_gate_up, None), linear_record(self.w_down, None), self.inner,
                          ops.activation_code(self.activation))

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        error_word = ctx.error_word if ctx is not None else None
        act = ops.gated_product(x, self.w_gate_up, self.inner, error_word, self.activation)
        return ops.linear(act, self.w_down, error_word=error_word, partial_ok=True)
