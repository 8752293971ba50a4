"""CUDA graphs for steps that hold decoded tokens only.

A decode step is a few hundred small launches; replayed from a graph it costs one launch
on the host.  A graph is captured per (row bucket, block-table width, key-split count per
group) with every index array in one static device buffer that is refilled by one copy
before each replay.  Rows beyond the live ones are padding: token 0 at position 0 whose
key and value go to the pool's spare page (the page after the last one the allocator
owns) and whose per-request state is the spare slot behind those that requests hold, so
they touch nothing that lives.  A mixer with state of its own may therefore be captured
too, if its step for decoded tokens runs on the device from ``ctx.state_slots`` alone.

The kernels, their arithmetic and the split of the keys are those of the eager path.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, Hashable, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .runner import AttentionLaunch, PagedBatch, StepContext, StepEntry, StepPlanner


def bucket_of(value: int, smallest: int = 1) -> int:
    bucket = smallest
    while bucket < value:
        bucket *= 2
    return bucket


@dataclass
class CapturedStep:
    graph: torch.cuda.CUDAGraph
    staging: torch.Tensor            # pinned int32, same layout as ``static``
    static: torch.Tensor             # device int32
    layout: Dict[str, Tuple[int, int]]
    logits: torch.Tensor             # [bucket, vocab] float32, rewritten by every replay
    keep: tuple                      # tensors the graph's kernels point at
    copied: Optional[torch.cuda.Event] = None   # the last copy out of ``staging``


class DecodeGraphs:
    MAX_ROWS = 256
    #: floats of split scratch that all captured steps share (they replay one after another); a step whose
    #: partial results do not fit runs its rows in several launches over it (the keys of a row are always
    #: cut at the same positions, whatever the batch)
    SCRATCH_FLOATS = 16 << 20
    #: captured steps kept; the one unused for longest goes first
    MAX_CAPTURED = 48
    #: bytes of logits that the kept steps may hold together (each owns [bucket, vocab] floats in the graphs'
    #: pool: 155 MB at 256 rows and a vocabulary of 152 k); beyond it the steps unused for longest go as well
    MAX_LOGIT_BYTES = 2 << 30

    def __init__(self, model, cache, planner: StepPlanner):
        self.model, self.cache, self.planner = model, cache, planner
        self.device, self.dtype = planner.device, planner.dtype
        self.captured: "OrderedDict[Hashable, CapturedStep]" = OrderedDict()
        self.pool = None
        self._scratch: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
        self.replays = 0
        self.kernels_per_replay: Dict[Hashable, int] = {}

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        if not (0 < len(entries) <= self.MAX_ROWS
                and all(len(e.tokens) == 1 and list(e.want) in ([], [0]) for e in entries)):
            return False
        # even one row's partial results must fit the shared scratch (else the step runs uncaptured)
        most = bucket_of(max(e.handle.length for e in entries) // StepPlanner.SPLIT_SIZE + 1)
        return most * max(self.planner._scratch_acc_width, 1) <= self.SCRATCH_FLOATS

    # ------------------------------------------------------------------ one step
    def run(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Entries are validated and their pages reserved.  Returns logits of the entries
        that want them, in order."""
        rows = len(entries)
        bucket = bucket_of(rows)
        groups = list(self.cache.allocators)
        page_size = self.cache.page_size
        stride = bucket_of(max([e.handle.table_length(key) for e in entries for key in groups] + [1]), 8)
        positions = np.fromiter((e.handle.length for e in entries), dtype=np.int64, count=rows)
        splits = []
        size = StepPlanner.SPLIT_SIZE
        for key in groups:
            window = self.cache.windows[key]
            begin = np.maximum(0, positions + 1 - window) if window else np.zeros_like(positions)
            splits.append(bucket_of(int((positions // size - begin // size + 1).max())))
        key = (bucket, stride, tuple(splits))
        step = self.captured.get(key)
        if step is None:
            step = self._prepare(key, groups)
            while len(self.captured) > self.MAX_CAPTURED:
                self.captured.popitem(last=False)
            while len(self.captured) > 1 and self._logit_bytes() > self.MAX_LOGIT_BYTES:
                self.captured.popitem(last=False)
        self.captured.move_to_end(key)
        if step.graph is None:
            # Captured, and run twice before that, on rows that are all padding: what those runs write goes to the
            # spare page and the spare state slot, so a mixer whose step is not idempotent (a running state) is
            # not stepped twice for the live requests.
            self._fill(step, [], groups, bucket, stride, positions, page_size)
            step.static.copy_(step.staging, non_blocking=True)
            self._capture(key, step, groups, bucket, stride, splits)
        if step.copied is not None:
            step.copied.synchronize()        # the staging buffer is free again once its last copy has run
        self._fill(step, entries, groups, bucket, stride, positions, page_size)
        step.static.copy_(step.staging, non_blocking=True)
        if any(e.token_from >= 0 for e in entries):
            # tokens that the step before chose and that never went to the host
            (t0, _), (f0, _) = step.layout["tokens"], step.layout["token_from"]
            ops.take_tokens(step.static[t0:t0 + rows], token_source, step.static[f0:f0 + rows], self.planner.error_word)
        self.planner.last_upload_bytes = step.staging.numel() * 4
        if step.copied is None:
            step.copied = torch.cuda.Event()
        step.copied.record()
        step.graph.replay()
        self.replays += 1
        ops.launch_count += self.kernels_per_replay[key]
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            return None
        if len(wanted) == rows:
            return step.logits[:rows]
        return step.logits[torch.tensor(wanted, device=self.device)]

    def _logit_bytes(self) -> int:
        return sum(step.logits.numel() * 4 for step in self.captured.values() if step.logits is not None)

    # ------------------------------------------------------------------ buffers
    def _prepare(self, key, groups) -> CapturedStep:
        bucket, stride = key[0], key[1]
        layout, offset = {}, 0
        for name, size in (("tokens", bucket), ("positions", bucket), ("row_request", bucket), ("cu_rows", bucket + 1),
                           ("state_slots", bucket), ("logit_rows", bucket), ("token_from", bucket)):
            layout[name] = (offset, size)
            offset += (size + 3) // 4 * 4
        for g in range(len(groups)):
            layout[f"table{g}"] = (offset, bucket * stride)
            offset += bucket * stride
            layout[f"slots{g}"] = (offset, bucket)
            offset += (bucket + 3) // 4 * 4
        staging = torch.zeros(offset, dtype=torch.int32, pin_memory=True)
        static = torch.zeros(offset, dtype=torch.int32, device=self.device)
        step = CapturedStep(None, staging, static, layout, None, ())
        self.captured[key] = step
        return step

    def _fill(self, step: CapturedStep, entries, groups, bucket, stride, positions, page_size) -> None:
        """The pinned copy of the step's index arrays, written by the C++ books."""
        names = ["tokens", "positions", "row_request", "cu_rows", "state_slots", "logit_rows", "token_from"]
        for g in range(len(groups)):
            names += [f"table{g}", f"slots{g}"]
        offsets = [step.layout[name][0] for name in names]
        self.cache.fill_decode([e.handle for e in entries], [int(e.tokens[0]) for e in entries],
                               [e.token_from for e in entries], bucket, stride, offsets, step.staging.numpy())

    # ------------------------------------------------------------------ capture
    def _context(self, step: CapturedStep, groups, bucket, stride, splits) -> Tuple[StepContext, torch.Tensor, list]:
        def part(name):
            begin, size = step.layout[name]
            return step.static[begin:begin + size]
        ctx = StepContext(self.device, self.dtype, bucket, bucket, part("tokens"), part("positions"),
                          part("row_request"), part("cu_rows"), part("state_slots"), self.planner.error_word,
                          host_cu_rows=list(range(bucket + 1)), host_start_positions=[0] * bucket,
                          host_state_slots=[0] * bucket)
        if self._scratch is None:
            width = max(self.planner._scratch_acc_width, 1)
            ml = max(self.SCRATCH_FLOATS // width * max(self.planner._scratch_ml_width, 1), 1)
            self._scratch = (torch.empty(self.SCRATCH_FLOATS, dtype=torch.float32, device=self.device),
                             torch.empty(ml, dtype=torch.float32, device=self.device))
        acc, ml = self._scratch
        keep = [acc, ml]
        size = StepPlanner.SPLIT_SIZE
        for g, key in enumerate(groups):
            # as many rows per launch as the scratch holds partial results for (bucket and count are powers of two)
            per_launch = bucket
            while per_launch > 1 and per_launch * splits[g] * max(self.planner._scratch_acc_width, 1) > self.SCRATCH_FLOATS:
                per_launch //= 2
            launches = [AttentionLaunch(first, first + per_launch, size, splits[g], None, None, splits[g] * size)
                        for first in range(0, bucket, per_launch)]
            ctx.paged[key] = PagedBatch(part(f"table{g}").view(bucket, stride), part(f"slots{g}"), launches, acc, ml,
                                        self.planner.counters)
        return ctx, part("logit_rows"), keep

    def _capture(self, key, step: CapturedStep, groups, bucket, stride, splits) -> None:
        ctx, logit_rows, keep = self._context(step, groups, bucket, stride, splits)
        caches = [self.cache.layer_cache(i) for i in range(len(self.model.program))]
        current = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(current)
        with torch.cuda.stream(side), ops.stream_scope():   # the same rows twice: libraries settle their workspaces
            for _ in range(2):
                self.model.forward(ctx, caches, logit_rows)
        current.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph, pool=self.pool), ops.stream_scope():
            logits = self.model.forward(ctx, caches, logit_rows)
        self.kernels_per_replay[key] = ops.launch_count - before
        if self.pool is None:
            self.pool = graph.pool()
        step.graph, step.logits, step.keep = graph, logits, (ctx, keep)
