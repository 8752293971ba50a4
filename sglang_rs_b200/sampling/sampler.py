"""From logits to one token per request.

Greedy and plain temperature sampling run in one kernel of this package (argmax; softmax of
l / T and an inverse-CDF walk in vocabulary order with the request's own uniform number), the
top-k / top-p / min-p cuts in another that follows the reference's algorithm
(crates/sglang-srt/src/model_executor.rs:471-555): sort descending; keep k; keep an item while
the mass before it is below top_p; drop items below max_p * min_p; walk the kept items in
sorted order with target = u * kept mass.  Penalties (model_executor.rs:558-590) change the logits of tokens
seen in prompt and output first, from counts kept on the device.  None of this needs a request's
tokens on the host, so steps overlap the host whatever the sampling options.

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


class SeenCounts:
    """How often each token occurred in the prompt and output of the requests that have penalties:
    one row of ``vocab`` counts per such request, on the device.  The prompt is counted when the
    request arrives, every sampled token by the sampler as it is chosen; the row goes back when the
    request ends."""

    def __init__(self, vocab: int, device):
        self.vocab, self.device = int(vocab), device
        self.table = None                       # int32 [capacity, vocab]
        self.rows = {}                          # request id -> row
        self.free = []

    def open(self, request_id, prompt: Sequence[int]) -> None:
        if not self.free:
            old = 0 if self.table is None else self.table.shape[0]
            grown = torch.zeros((max(4, 2 * old), self.vocab), dtype=torch.int32, device=self.device)
            if old:
                grown[:old].copy_(self.table)
            self.table = grown
            self.free = list(range(grown.shape[0] - 1, old - 1, -1))
        row = self.free.pop()
        self.rows[request_id] = row
        self.table[row].zero_()
        if len(prompt):
            tokens = torch.tensor(list(prompt), dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            ops.count_tokens(self.table[row], tokens)

    def close(self, request_id) -> None:
        row = self.rows.pop(request_id, None)
        if row is not None:
            self.free.append(row)

    def row_of(self, request_id) -> int:
        return self.rows.get(request_id, -1)


class Sampler:
    def __init__(self, device, vocab: int = 0):
        self.device = device
        self.seen = SeenCounts(vocab, device)

    def pick_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                       randoms: Sequence[RequestRandom], request_ids: Sequence = ()) -> torch.Tensor:
        """One token per row: the chosen ids stay on the device (int32 [rows]); nothing waits for the
        GPU.  ``request_ids`` name the rows' requests, for those with penalties (``logits`` is then
        changed in place, and the chosen tokens are counted as seen)."""
        rows = logits.shape[0]
        penalised = [r for r in range(rows) if params[r].has_penalties]
        # what the kernels need per row, in one tensor of floats and one of ints: two copies per step at most
        temperature, uniform = [0.0] * rows, [0.0] * rows          # of the rows sampled without cuts
        cut_temperature, top_p, min_p = [1.0] * rows, [1.0] * rows, [0.0] * rows
        presence, frequency, repetition = [0.0] * rows, [0.0] * rows, [1.0] * rows
        top_k, seen_row = [0] * rows, [-1] * rows
        cut = []                                                   # rows with top-k / top-p / min-p
        for r, p in enumerate(params):
            if p.has_penalties:
                seen_row[r] = self.seen.row_of(request_ids[r]) if r < len(request_ids) else -1
                if seen_row[r] < 0:
                    raise RuntimeError("a request with penalties has no row of counts; SeenCounts.open was not called")
                presence[r], frequency[r] = p.presence_penalty or 0.0, p.frequency_penalty or 0.0
                repetition[r] = p.repetition_penalty if p.repetition_penalty is not None else 1.0
            if p.is_greedy:
                continue
            uniform[r] = randoms[r].next_unit()
            if p.filters:
                cut.append(r)
                cut_temperature[r] = p.effective_temperature
                top_k[r] = int(p.top_k) if p.top_k is not None else 0
                top_p[r] = float(p.top_p) if p.top_p is not None else 1.0
                min_p[r] = float(p.min_p) if p.min_p is not None else 0.0
            else:
                temperature[r] = p.effective_temperature
        plain = any(t > 0 for t in temperature)
        floats = ints = None
        if plain or cut or penalised:
            floats = torch.tensor([temperature, uniform, cut_temperature, top_p, min_p, presence, frequency, repetition],
                                  dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        if cut or penalised:
            ints = torch.tensor([top_k, seen_row, cut + [0] * (rows - len(cut))],
                                dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        if penalised:
            ops.apply_penalties(logits, self.seen.table, ints[1], floats[5], floats[6], floats[7])
        if len(cut) == rows:
            picked = torch.empty(rows, dtype=torch.int32, device=logits.device)      # every row is written below
        elif plain:
            picked = ops.sample(logits, floats[0], floats[1])
        else:
            picked = ops.sample(logits, None, None)
        if cut:
            ops.sample_filtered(logits, ints[2, :len(cut)], floats[2], ints[0], floats[3], floats[4], floats[1], picked)
        if penalised:
            ops.count_picked(self.seen.table, ints[1], picked)
        return picked

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], randoms: Sequence[RequestRandom],
               request_ids: Sequence = ()) -> List[int]:
        """The same with the chosen token ids brought to the host."""
        return self.pick_on_device(logits, params, randoms, request_ids).cpu().tolist()
