"""From logits to one token per request.

Greedy and plain temperature sampling run in this package's kernel (argmax; softmax of
l / T and an inverse-CDF walk in vocabulary order with the request's own uniform number).
Penalties and the top-k / top-p / min-p cuts follow the reference's algorithm
(crates/sglang-srt/src/model_executor.rs:449-590) with tensor operations on the device:
penalise tokens seen in prompt and output; sort descending; keep k; keep an item while
the mass before it is below top_p; drop items below max_p * min_p; walk the kept items in
sorted order with target = u * kept mass.

Each request draws from its own generator, seeded by its ``seed`` (or by its id), so its
tokens do not depend on what else is in the batch.
"""
from __future__ import annotations

import random
import zlib
from typing import List, Sequence

import torch

from .. import ops
from .params import SamplingParams

ONE_BELOW = 1.0 - 2.0 ** -24      # the reference clamps u to [0, 1 - 2^-24] (model_executor.rs:548-555)


class RequestRandom:
    """The request's stream of uniform numbers in [0, 1)."""

    def __init__(self, request_id, seed):
        key = seed if seed is not None else zlib.crc32(repr(request_id).encode("utf-8"))
        self._generator = random.Random(int(key))

    def next_unit(self) -> float:
        return min(max(self._generator.random(), 0.0), ONE_BELOW)


def apply_penalties(row: torch.Tensor, seen: Sequence[int], params: SamplingParams) -> torch.Tensor:
    """Penalised copy of a logits row (model_executor.rs:558-590)."""
    out = row.clone()
    if not seen:
        return out
    tokens = torch.as_tensor(list(seen), dtype=torch.long, device=row.device)
    tokens = tokens[tokens < row.numel()]
    unique, counts = torch.unique(tokens, return_counts=True)
    values = out[unique]
    repetition = params.repetition_penalty if params.repetition_penalty is not None else 1.0
    if repetition != 1.0:
        values = torch.where(values < 0, values * repetition, values / repetition)
    values = values - (params.presence_penalty or 0.0) - (params.frequency_penalty or 0.0) * counts.to(values.dtype)
    out[unique] = values
    return out


def sample_filtered(row: torch.Tensor, params: SamplingParams, u: float) -> int:
    """top-k / top-p / min-p on one row (model_executor.rs:471-546)."""
    scaled = row / params.effective_temperature
    probs = torch.exp(scaled - scaled.max())
    probs, order = torch.sort(probs, descending=True, stable=True)
    if params.top_k is not None and 0 < params.top_k < probs.numel():
        probs, order = probs[:params.top_k], order[:params.top_k]
    total = probs.sum()
    before = torch.cumsum(probs / total, dim=0) - probs / total          # mass before each item
    keep = (before < (1.0 if params.top_p is None else params.top_p)) & (probs >= probs[0] * (params.min_p or 0.0))
    kept, kept_order = probs[keep], order[keep]
    running = torch.cumsum(kept, dim=0)
    target = u * float(running[-1])
    index = int(torch.searchsorted(running, torch.tensor(target, device=row.device, dtype=running.dtype), right=True))
    return int(kept_order[min(index, kept.numel() - 1)])


class Sampler:
    def __init__(self, device):
        self.device = device

    def pick_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                       randoms: Sequence[RequestRandom]) -> torch.Tensor:
        """Greedy and plain temperature rows only (no penalties, no top-k / top-p / min-p): the
        chosen ids stay on the device (int32 [rows]); nothing waits for the GPU."""
        rows = logits.shape[0]
        temperature = [0.0] * rows
        uniform = [0.0] * rows
        for r, p in enumerate(params):
            if not p.is_greedy:
                uniform[r] = randoms[r].next_unit()
                temperature[r] = p.effective_temperature
        if any(t > 0 for t in temperature):
            staged = torch.tensor([temperature, uniform], dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
            return ops.sample(logits, staged[0].contiguous(), staged[1].contiguous())
        return ops.sample(logits, None, None)

    @staticmethod
    def stays_on_device(params: SamplingParams) -> bool:
        """True if :meth:`pick_on_device` samples this request exactly as :meth:`sample` does."""
        return not params.has_penalties and (params.is_greedy or not params.filters)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[RequestRandom],
               seen_tokens: Sequence[Sequence[int]]) -> List[int]:
        """``logits`` [rows, vocab] float32 on the device; one entry of the other arguments
        per row.  Returns the chosen token ids on the host."""
        rows = logits.shape[0]
        if any(p.has_penalties for p in params):
            logits = logits.clone()
            for r, p in enumerate(params):
                if p.has_penalties:
                    logits[r] = apply_penalties(logits[r], seen_tokens[r], p)
        temperature = [0.0] * rows
        uniform = [0.0] * rows
        slow = []
        for r, p in enumerate(params):
            if p.is_greedy:
                continue
            uniform[r] = randoms[r].next_unit()
            if p.filters:
                slow.append(r)
            else:
                temperature[r] = p.effective_temperature
        if any(t > 0 for t in temperature):
            staged = torch.tensor([temperature, uniform], dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
            picked = ops.sample(logits, staged[0].contiguous(), staged[1].contiguous())
        else:
            picked = ops.sample(logits, None, None)
        tokens = picked.cpu().tolist()
        for r in slow:
            tokens[r] = sample_filtered(logits[r], params[r], uniform[r])
        return tokens
