"""The step function: one batch of (request, its next tokens) through the model.

A step runs only the tokens it is given, from the cache that earlier steps left, and
returns 32-bit logits at the rows that were asked for.  Prompt portions and single decoded
tokens sit side by side in the flat row arrays; nothing below the flattening knows a
"prefill" from a "decode" (the reference's flat batch already has this shape:
crates/sglang-srt/src/model_executor.rs:16-33, with positions that need not start at 0,
:172-173, and causality by length, crates/sglang-srt/src/cuda_attention.rs:285-297).

Both generation (the scheduler) and trace replay call :meth:`ModelRunner.step`.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, OutOfPages, RequestCache
from ..ops import trace
from .metrics import StepLog, StepStats, step_log_target


class StepInputError(ValueError):
    """A step that cannot run: bad token id, position past the model's limit, bad index."""


@dataclass
class StepEntry:
    handle: RequestCache
    tokens: Sequence[int]
    #: indices into ``tokens`` whose logits are wanted
    want: Sequence[int] = ()
    #: >= 0: the entry's single token is not known on the host; it is row ``token_from`` of the
    #: ``token_source`` tensor given to the step (what the step before chose, still on the device)
    token_from: int = -1


@dataclass
class AttentionLaunch:
    """Rows [begin, end) of the step run as one launch.  ``split_size`` 0: one block walks
    all keys of a row; else the keys are cut every ``split_size`` positions."""
    begin: int
    end: int
    split_size: int
    max_splits: int
    #: for an unsplit launch: int32 [tiles, 4] = (first row, rows, request, first position), rows in tiles
    #: of at most ``StepPlanner.TILE_ROWS`` consecutive rows of one request
    tiles: Optional[torch.Tensor] = None
    #: the same rows cut into tiles of at most ``StepPlanner.WIDE_TILE_ROWS`` (for the tcgen05 kernel)
    wide_tiles: Optional[torch.Tensor] = None
    #: for a split launch: the most keys any of its rows sees (a bound is enough)
    max_keys: Optional[int] = None


@dataclass
class PagedBatch:
    """Per-step view of one cache group."""
    block_table: torch.Tensor            # int32 [requests, stride]
    slots: torch.Tensor                  # int32 [rows]: where each row's key and value go
    launches: List[AttentionLaunch]
    scratch_acc: Optional[torch.Tensor] = None
    scratch_ml: Optional[torch.Tensor] = None
    #: zeroed ints with which the blocks of a split run find out which of them merges the splits
    counters: Optional[torch.Tensor] = None


@dataclass
class StepContext:
    device: torch.device
    dtype: torch.dtype
    num_rows: int
    num_requests: int
    token_ids: torch.Tensor              # int32 [rows]
    positions: torch.Tensor              # int32 [rows]
    row_request: torch.Tensor            # int32 [rows]: index into this step's requests
    cu_rows: torch.Tensor                # int32 [requests + 1]: rows of request r are cu_rows[r] .. cu_rows[r+1]
    state_slots: torch.Tensor            # int32 [requests]
    error_word: torch.Tensor
    paged: Dict[Hashable, PagedBatch] = field(default_factory=dict)
    # host mirrors, for parts that plan on the host
    host_cu_rows: Sequence[int] = ()
    host_start_positions: Sequence[int] = ()
    host_state_slots: Sequence[int] = ()


class StepPlanner:
    """Turns a step's entries into the flat device arrays and the per-group plans that the
    parts read.  It needs the cache manager and the scratch widths of the mixers, not the
    model, so a single part can be stepped with it."""
    #: keys per split of a decode row; fixed, so a row's arithmetic depends on its own position only
    SPLIT_SIZE = 128
    #: a request that brings at most this many rows is run with split keys
    SPLIT_ROWS_PER_REQUEST = 1
    #: rows of one request that the tiled attention kernel takes per block
    TILE_ROWS = 64
    WIDE_TILE_ROWS = 128
    #: floats of attention scratch above which the decoded rows of a step go in several launches
    SCRATCH_LIMIT = 64 << 20

    def __init__(self, cache: CacheManager, device, dtype: torch.dtype, scratch_widths: Sequence = ()):
        self.cache, self.device, self.dtype = cache, torch.device(device), dtype
        self.error_word = ops.new_error_word(self.device)
        # floats of split scratch per (row, split) that the widest mixer needs
        self._scratch_acc_width = max((w[0] for w in scratch_widths), default=0)
        self._scratch_ml_width = max((w[1] for w in scratch_widths), default=0)
        self._scratch: Dict[str, torch.Tensor] = {}
        self.counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        self.last_upload_bytes = 0

    # ------------------------------------------------------------------ flattening
    def flatten(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None):
        # decoded tokens first, portions after them: each kind is one contiguous row range
        order = sorted(range(len(entries)),
                       key=lambda i: (len(entries[i].tokens) > self.SPLIT_ROWS_PER_REQUEST, i))
        starts = [0] * len(entries)
        cu_rows = [0]
        tokens: List[int] = []
        token_from: List[int] = []
        positions: List[int] = []
        row_request: List[int] = []
        start_positions: List[int] = []
        state_slots: List[int] = []
        split_rows = 0
        for slot, index in enumerate(order):
            entry = entries[index]
            count = len(entry.tokens)
            starts[index] = cu_rows[-1]
            tokens.extend(int(t) for t in entry.tokens)
            token_from.extend([entry.token_from] * count)
            positions.extend(range(entry.handle.length, entry.handle.length + count))
            row_request.extend([slot] * count)
            start_positions.append(entry.handle.length)
            state_slots.append(entry.handle.state_slot)
            cu_rows.append(cu_rows[-1] + count)
            if count <= self.SPLIT_ROWS_PER_REQUEST:
                split_rows = cu_rows[-1]
        rows = cu_rows[-1]
        logit_rows = [starts[i] + int(w) for i, entry in enumerate(entries) for w in entry.want]

        groups = list(self.cache.allocators)
        ordered = [entries[index].handle for index in order]
        counts = [len(entries[index].tokens) for index in order]
        stride = 1
        for handle in ordered:
            for key in groups:
                stride = max(stride, handle.table_length(key))
        tables, slots = {}, {}
        for key in groups:
            tables[key], slots[key] = self.cache.fill_group(key, ordered, counts, stride)   # from the C++ books

        tiles: List[int] = []
        wide_tiles: List[int] = []
        for slot in range(len(order)):
            if cu_rows[slot] < split_rows:
                continue
            for size, into in ((self.TILE_ROWS, tiles), (self.WIDE_TILE_ROWS, wide_tiles)):
                for first in range(cu_rows[slot], cu_rows[slot + 1], size):
                    into += [first, min(size, cu_rows[slot + 1] - first), slot,
                             start_positions[slot] + first - cu_rows[slot]]
        # tiles with the most keys first: the blocks that work longest start first
        def by_falling_work(flat: List[int]) -> np.ndarray:
            table = np.asarray(flat, dtype=np.int32).reshape(-1, 4)
            return table[np.argsort(-(table[:, 1] + table[:, 3]), kind="stable")].reshape(-1)
        tiles, wide_tiles = by_falling_work(tiles), by_falling_work(wide_tiles)
        pieces = [np.asarray(tokens, dtype=np.int32), np.asarray(positions, dtype=np.int32),
                  np.asarray(row_request, dtype=np.int32), np.asarray(cu_rows, dtype=np.int32),
                  np.asarray(state_slots, dtype=np.int32), np.asarray(logit_rows, dtype=np.int32),
                  np.asarray(tiles, dtype=np.int32), np.asarray(wide_tiles, dtype=np.int32)]
        for key in groups:
            pieces.append(tables[key].reshape(-1))
            pieces.append(slots[key])
        from_device = any(f >= 0 for f in token_from)
        if from_device:
            pieces.append(np.asarray(token_from, dtype=np.int32))
        device_pieces = self._upload(pieces)
        if from_device:
            ops.take_tokens(device_pieces[0], token_source, device_pieces[-1], self.error_word)
        (token_ids, positions_d, row_request_d, cu_rows_d, state_slots_d, logit_rows_d, tiles_d,
         wide_tiles_d) = device_pieces[:8]
        tiles_d, wide_tiles_d = tiles_d.view(-1, 4), wide_tiles_d.view(-1, 4)

        ctx = StepContext(self.device, self.dtype, rows, len(order), token_ids, positions_d, row_request_d,
                          cu_rows_d, state_slots_d, self.error_word, host_cu_rows=cu_rows,
                          host_start_positions=start_positions, host_state_slots=state_slots)
        np_positions = np.asarray(positions, dtype=np.int64)
        for g, key in enumerate(groups):
            table_d = device_pieces[8 + 2 * g].view(len(order), stride)
            slots_d = device_pieces[9 + 2 * g]
            ctx.paged[key] = self._plan(key, table_d, slots_d, np_positions, split_rows, rows, tiles_d, wide_tiles_d)
        return ctx, (logit_rows_d if logit_rows else None)

    def _upload(self, pieces: Sequence[np.ndarray]) -> List[torch.Tensor]:
        """All of a step's index arrays in one pinned buffer and one copy."""
        sizes = [piece.size for piece in pieces]
        offsets = np.concatenate([[0], np.cumsum([(size + 3) // 4 * 4 for size in sizes])])
        total = int(offsets[-1])
        staging = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=True)
        view = staging.numpy()
        for piece, offset, size in zip(pieces, offsets, sizes):
            view[offset:offset + size] = piece
        self.last_upload_bytes = total * 4
        on_device = staging.to(self.device, non_blocking=True)
        return [on_device[offset:offset + size] for offset, size in zip(offsets[:-1], sizes)]

    def _plan(self, key, table_d, slots_d, positions: np.ndarray, split_rows: int, rows: int,
              tiles_d: Optional[torch.Tensor] = None, wide_tiles_d: Optional[torch.Tensor] = None) -> PagedBatch:
        window = self.cache.windows[key]
        launches: List[AttentionLaunch] = []
        scratch_acc = scratch_ml = None
        if split_rows > 0:
            pos = positions[:split_rows]
            begin = np.maximum(0, pos + 1 - window) if window else np.zeros_like(pos)
            split_size = self.SPLIT_SIZE
            per_row = pos // split_size - begin // split_size + 1
            visible_per_row = pos + 1 - begin
            # The keys are always cut every SPLIT_SIZE positions, so a row's arithmetic is a function of its
            # own position.  When the partial results of all rows do not fit the scratch memory, the rows go
            # in several launches, one after another over the same scratch, never in longer pieces.
            width = max(self._scratch_acc_width, 1)
            rows_per_launch = max(1, self.SCRATCH_LIMIT // (int(per_row.max()) * width))
            need_acc = need_ml = 0
            for first in range(0, split_rows, rows_per_launch):
                last = min(split_rows, first + rows_per_launch)
                max_splits = int(per_row[first:last].max())
                visible = int(visible_per_row[first:last].max())
                # the split count of the generic kernel, or that of the tensor-core decode kernel if larger
                # (as far as the scratch limit lets it go)
                fit = max(1, self.SCRATCH_LIMIT // ((last - first) * width))
                widest = max(max_splits, min(ops.decode_splits_bound(visible), fit))
                need_acc = max(need_acc, (last - first) * widest * self._scratch_acc_width)
                need_ml = max(need_ml, (last - first) * widest * self._scratch_ml_width)
                launches.append(AttentionLaunch(first, last, split_size, max_splits, None, None, visible))
            scratch_acc = self._scratch_tensor("acc", need_acc)
            scratch_ml = self._scratch_tensor("ml", need_ml)
        if rows > split_rows:
            launches.append(AttentionLaunch(split_rows, rows, 0, 1, tiles_d, wide_tiles_d))
        return PagedBatch(table_d, slots_d, launches, scratch_acc, scratch_ml, self.counters)

    def _scratch_tensor(self, name: str, floats: int) -> torch.Tensor:
        current = self._scratch.get(name)
        if current is None or current.numel() < floats:
            current = torch.empty(max(floats, 1), dtype=torch.float32, device=self.device)
            self._scratch[name] = current
        return current


class ModelRunner:
    def __init__(self, model, cache: CacheManager, use_cuda_graphs: bool = True, native_step: Optional[bool] = None):
        if model.device is None:
            raise RuntimeError("the model has no weights yet")
        if model.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no host path")
        ops.require_supported_device(model.device)
        self.model, self.cache = model, cache
        self.device, self.dtype = model.device, model.dtype
        widths = [layer.split_scratch() for layer in model.layers if hasattr(layer, "split_scratch")]
        self.planner = StepPlanner(cache, self.device, self.dtype, widths)
        self.error_word = self.planner.error_word
        self.steps_run = 0
        #: the record of the last step, and the log that keeps (and, if asked by SRB_STEP_LOG, writes) them all
        self.last_stats: Optional[StepStats] = None
        self.step_log = StepLog(step_log_target())
        # A model whose parts all have records for the step executor runs a step in one native call
        # (``native_step`` False, or SRB_NATIVE_STEP=0, keeps the part-by-part launches).
        if native_step is None:
            native_step = os.environ.get("SRB_NATIVE_STEP", "1") not in ("0", "off", "false")
        model.native = None
        if native_step:
            from .native import NativeModel, prepare
            model.native = NativeModel.of(model)
            if model.native is not None:
                prepare(model.native, cache.page_size)
        self.graphs = None
        if use_cuda_graphs and all(getattr(layer, "graph_safe", False) for layer in model.layers):
            from .graphs import DecodeGraphs
            self.graphs = DecodeGraphs(model, cache, self.planner)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns logits [wanted rows, vocab] (float32, on the device) in
        the order of ``entries`` and of each entry's ``want``, or None if none is wanted.
        ``token_source``: int32 on the device, read by entries with ``token_from`` set."""
        entries = [entry for entry in entries]
        if not entries:
            return None
        started = time.perf_counter()
        timers = trace.active
        begin = end = None
        if self.step_log.time_device or (timers is not None and timers.events):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
        self._validate(entries, token_source)
        reserved: List[StepEntry] = []
        try:
            for entry in entries:
                self.cache.reserve(entry.handle, len(entry.tokens))
                reserved.append(entry)
        except OutOfPages:
            for entry in reserved:
                self.cache.trim_reservation(entry.handle)
            raise
        captured = False
        try:
            if self.graphs is not None and self.graphs.eligible(entries):
                logits = self.graphs.run(entries, token_source)
                captured = True
            else:
                ctx, logit_rows = self.planner.flatten(entries, token_source)
                caches = [self.cache.layer_cache(i) for i in range(len(self.model.program))]
                with ops.stream_scope():
                    logits = self.model.forward(ctx, caches, logit_rows)
        except Exception:
            for entry in entries:
                self.cache.trim_reservation(entry.handle)
            raise
        for entry in entries:
            self.cache.commit(entry.handle, len(entry.tokens))
        self.steps_run += 1
        if end is not None:
            end.record()
        counts = [len(entry.tokens) for entry in entries]
        decode_rows = sum(1 for count in counts if count == 1)
        stats = StepStats(
            step=self.steps_run, rows=sum(counts), requests=len(entries), decode_rows=decode_rows,
            prompt_rows=sum(counts) - decode_rows, wanted=sum(len(entry.want) for entry in entries), captured=captured,
            pages_free={":".join(str(part) for part in key) if isinstance(key, tuple) else str(key): free
                        for key, free in self.cache.free_pages().items()},
            host_ms=(time.perf_counter() - started) * 1e3)
        if timers is not None and timers.events:
            stats.kernels = {kind: round(ms, 4) for kind, ms in timers.collect().items()}    # waits for the step
        self.step_log.add(stats, begin, end)
        self.last_stats = stats
        return logits

    def check_device_errors(self) -> None:
        """Reads the device-side error word (a synchronisation) and raises if a kernel
        skipped an access."""
        ops.raise_on_error_word(self.error_word)

    def raise_on_error_bits(self, value: int) -> None:
        """The same check for a copy of the error word that is on the host already."""
        ops.raise_on_error_value(int(value), self.error_word)

    # ------------------------------------------------------------------ checks
    def _validate(self, entries: Sequence[StepEntry], token_source: Optional[torch.Tensor] = None) -> None:
        seen = set()
        for entry in entries:
            handle = entry.handle
            if handle.closed:
                raise StepInputError(f"request {handle.request_id!r} has ended")
            if id(handle) in seen:
                raise StepInputError(f"request {handle.request_id!r} appears twice in one step")
            seen.add(id(handle))
            count = len(entry.tokens)
            if count == 0:
                raise StepInputError(f"request {handle.request_id!r} brings no tokens")
            if handle.length + count > self.model.max_positions:
                raise StepInputError(
                    f"request {handle.request_id!r}: position {handle.length + count - 1} exceeds "
                    f"max_position_embeddings {self.model.max_positions}")
            if entry.token_from >= 0:
                if count != 1 or token_source is None or entry.token_from >= token_source.numel():
                    raise StepInputError(f"request {handle.request_id!r}: a token taken from the device must be the "
                                         f"entry's only one and lie inside the source")
            elif min(entry.tokens) < 0 or max(entry.tokens) >= self.model.vocab_size:
                raise StepInputError(f"request {handle.request_id!r}: a token id among {list(entry.tokens)[:8]}... is "
                                     f"outside the vocabulary of {self.model.vocab_size}")
            for index in entry.want:
                if not 0 <= int(index) < count:
                    raise StepInputError(f"request {handle.request_id!r}: wanted row {index} is not among its "
                                         f"{count} tokens")

