"""From logits to one token per request.

Greedy and plain temperature sampling run in one kernel of this package (argmax; softmax of
l / T and an inverse-CDF walk in vocabulary order with the request's own uniform number), the
top-k / top-p / min-p cuts in another that follows the reference's algorithm
(crates/sglang-srt/src/model_executor.rs:471-555): sort descending; keep k; keep an item while
the mass before it is below top_p; drop items below max_p * min_p; walk the kept items in
sorted order with target = u * kept mass.  Neither needs the request's tokens on the host, so
steps with such requests still overlap the host.  Penalties (model_executor.rs:558-590) change
the logits of tokens seen in prompt and output with tensor operations first.

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


class Sampler:
    def __init__(self, device):
        self.device = device

    def pick_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                       randoms: Sequence[RequestRandom]) -> torch.Tensor:
        """One token per row (penalties apart): the chosen ids stay on the device (int32 [rows]);
        nothing waits for the GPU."""
        rows = logits.shape[0]
        temperature = [0.0] * rows
        uniform = [0.0] * rows
        cut = []                                   # rows with top-k / top-p / min-p
        for r, p in enumerate(params):
            if p.is_greedy:
                continue
            uniform[r] = randoms[r].next_unit()
            if p.filters:
                cut.append(r)
            else:
                temperature[r] = p.effective_temperature
        staged = None
        if cut or any(t > 0 for t in temperature):
            floats = [temperature, uniform]
            if cut:
                floats += [[params[r].effective_temperature if params[r].filters and not params[r].is_greedy else 1.0
                            for r in range(rows)],
                           [float(params[r].top_p) if params[r].top_p is not None else 1.0 for r in range(rows)],
                           [float(params[r].min_p) if params[r].min_p is not None else 0.0 for r in range(rows)]]
            staged = torch.tensor(floats, dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        if staged is not None and any(t > 0 for t in temperature):
            picked = ops.sample(logits, staged[0], staged[1])
        else:
            picked = ops.sample(logits, None, None)
        if cut:
            ints = torch.tensor([[int(params[r].top_k) if params[r].top_k is not None else 0 for r in range(rows)],
                                 cut + [0] * (rows - len(cut))], dtype=torch.int32).pin_memory().to(self.device,
                                                                                                  non_blocking=True)
            ops.sample_filtered(logits, ints[1, :len(cut)], staged[2], ints[0], staged[3], staged[4], staged[1], picked)
        return picked

    @staticmethod
    def stays_on_device(params: SamplingParams) -> bool:
        """True if :meth:`pick_on_device` samples this request exactly as :meth:`sample` does."""
        return not params.has_penalties

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[RequestRandom],
               seen_tokens: Sequence[Sequence[int]]) -> List[int]:
        """``logits`` [rows, vocab] float32 on the device; one entry of the other arguments
        per row.  Returns the chosen token ids on the host."""
        if any(p.has_penalties for p in params):
            logits = logits.clone()
            for r, p in enumerate(params):
                if p.has_penalties:
                    logits[r] = apply_penalties(logits[r], seen_tokens[r], p)
        return self.pick_on_device(logits, params, randoms).cpu().tolist()
