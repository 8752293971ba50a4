"""Token embedding and output head.

h0 = embed[token] without scaling; logits = norm(h) . W_out^T with W_out the head's own
matrix or, if tied, the embedding table (reference:
crates/sglang-srt/src/cpu_reference.rs:741-752, :176-185).  Logits are 32-bit in every mode.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from .base import Part, TensorSpec, matrix_to


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab: int, width: int, weight_name: str):
        self.vocab, self.width, self.weight_name = int(vocab), int(width), weight_name
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width))}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.table = matrix_to(tensors[self.weight_name], device, dtype)

    def native_record(self):
        """The step executor reads the table itself; the record says only that there is one."""
        return None if self.table is None else True

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        residual = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        ops.embedding(token_ids, self.table, residual, ctx.error_word)
        return residual


class OutputHead(Part):
    """``weight_name`` None ties the head to ``embedding``'s table."""
    graph_safe = True


    def __init__(self, vocab: int, width: int, weight_name: Optional[str], embedding: Optional[TokenEmbedding] = None):
        if weight_name is None and embedding is None:
            raise ValueError("a tied head needs the embedding it shares")
        self.vocab, self.width, self.weight_name, self.embedding = int(vocab), int(width), weight_name, embedding
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.weight_name: TensorSpec((self.vocab, self.width))} if self.weight_name else {}

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        if self.weight_name:
            self.weight = matrix_to(tensors[self.weight_name], device, dtype)

    def native_record(self):
        weight = self.weight if self.weight_name else self.embedding.table
        return None if weight is None else True

    def forward(self, ctx, normed: torch.Tensor) -> torch.Tensor:
        weight = self.weight if self.weight_name else self.embedding.table
        return ops.linear(normed, weight, out_dtype=torch.float32, error_word=ctx.error_word)
