"""Arrangement of the parts of one layer.

Pre-norm residual form (reference: crates/sglang-srt/src/cpu_reference.rs:257-317):
h' = h + mixer(norm_1(h)); h'' = h' + feed_forward(norm_2(h')).  The hidden state travels
as (residual, delta) with h = residual + delta; each norm takes the pending sum first, in
32-bit, so no separate add kernel runs.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, Part, TensorSpec


class PreNormBlock(Part):
    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, feed_forward: FeedForward):
        self.input_norm, self.mixer, self.post_norm, self.feed_forward = input_norm, mixer, post_norm, feed_forward

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def parts(self):
        return (self.input_norm, self.mixer, self.post_norm, self.feed_forward)

    def cache_need(self):
        return self.mixer.cache_need()

    def split_scratch(self):
        return self.mixer.split_scratch()

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.parts():
            part.load(tensors, device, dtype)

    def native_record(self):
        """This block for the step executor, if each of its parts has a record of the kind the executor's
        pre-norm block is made of; else None, and the block runs part by part."""
        from ..ops.records import SxAttention, SxBlock, SxGatedMlp, SxNorm
        found = [part.native_record() if hasattr(part, "native_record") else None for part in self.parts()]
        kinds = (SxNorm, SxAttention, SxNorm, SxGatedMlp)
        if not all(isinstance(record, kind) for record, kind in zip(found, kinds)):
            return None
        return SxBlock(*found)

    def forward(self, ctx, cache, residual: torch.Tensor,
                delta: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        normed = self.input_norm.add_norm(residual, delta, ctx.dtype)
        delta = self.mixer.forward(ctx, cache, normed)
        normed = self.post_norm.add_norm(residual, delta, ctx.dtype)
        delta = self.feed_forward.forward(ctx, normed)
        return residual, delta
