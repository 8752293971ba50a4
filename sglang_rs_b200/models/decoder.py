"""A decoder model as data: parts, and the order in which they run.

``layers`` holds the blocks (each with its own weights); ``program`` is the list of layer
calls of one forward pass.  By default it is every layer once, in order, each with a cache
of its own (reference: crates/sglang-srt/src/cpu_reference.rs:152-174).  A program may call
a layer twice (two calls, two caches, one set of weights), and a call may read the cache
of an earlier call instead of keeping one (it then writes nothing).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from ..ops import trace
from ..parts.base import CacheNeed, Part, TensorSpec


@dataclass(frozen=True)
class LayerCall:
    layer: int
    #: index of an earlier call of the program whose cache this call reads; None = its own
    cache_from: Optional[int] = None


class DecoderModel(Part):
    def __init__(self, embedding, layers: Sequence, final_norm, head, *, vocab_size: int, max_positions: int,
                 program: Optional[Sequence[LayerCall]] = None, eos_token_ids: Sequence[int] = (),
                 ignored_tensors: Sequence[str] = ()):
        self.embedding, self.layers, self.final_norm, self.head = embedding, list(layers), final_norm, head
        self.vocab_size, self.max_positions = int(vocab_size), int(max_positions)
        self.eos_token_ids = tuple(eos_token_ids)
        #: shell-style patterns of checkpoint tensors that may be present and that nothing reads
        self.ignored_tensors = tuple(ignored_tensors)
        self.program: List[LayerCall] = list(program) if program is not None else [
            LayerCall(i) for i in range(len(self.layers))]
        for index, call in enumerate(self.program):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"program entry {index} names layer {call.layer}, which does not exist")
            if call.cache_from is not None:
                if not 0 <= call.cache_from < index or self.program[call.cache_from].cache_from is not None:
                    raise ValueError(f"program entry {index} must read the cache of an earlier call that owns one")
                theirs = self.layers[self.program[call.cache_from].layer].cache_need()
                if theirs != self.layers[call.layer].cache_need():
                    raise ValueError(f"program entry {index} reads a cache of another shape than its own")
        self.dtype: Optional[torch.dtype] = None
        self.device = None
        #: the model's records for the step executor (engine/native.py), set by the runner when every part has
        #: one; ``forward`` then is one native call
        self.native = None

    def all_parts(self):
        return [self.embedding, *self.layers, self.final_norm, self.head]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs: Dict[str, TensorSpec] = {}
        for part in self.all_parts():
            specs.update(part.tensor_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        for part in self.all_parts():
            part.load(tensors, device, dtype)
        self.device, self.dtype = torch.device(device), dtype

    def cache_needs(self) -> List[CacheNeed]:
        """One entry per program call; a call that reads another's cache needs none."""
        return [None if call.cache_from is not None else self.layers[call.layer].cache_need()
                for call in self.program]

    def forward(self, ctx, caches: Sequence, logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the rows of ``ctx``; returns 32-bit logits of the rows in ``logit_rows``
        (None or empty: the pass only fills the caches)."""
        if self.native is not None and trace.active is None and all(
                cache is not None and hasattr(cache, "k_pool") for cache in caches):
            return self.native.run(ctx, caches, logit_rows)
        residual = self.embedding.forward(ctx, ctx.token_ids)
        delta = None
        for index, call in enumerate(self.program):
            cache = caches[index if call.cache_from is None else call.cache_from]
            if call.cache_from is not None and cache is not None:
                cache = cache.read_only()
            residual, delta = self.layers[call.layer].forward(ctx, cache, residual, delta)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        normed = self.final_norm.add_norm(residual, delta, ctx.dtype, row_index=logit_rows)
        return self.head.forward(ctx, normed)
