"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

What it keeps of the reference (crates/sglang-srt/src/scheduler.rs): first come, first
served admission (:463-510) under ``max_running_requests`` (:512-525); a token budget per
step that counts only tokens still to be computed (:484-494); the first request is taken
even if it alone exceeds the budget, here cut to the budget instead (:497-507); a request
finishes on a stop token, which stays in its output, unless ``ignore_eos``
(crates/sglang-srt/src/model_executor.rs:763-769), or when ``max_new_tokens`` are out
(:195-197, :821); abort by id releases the request's pages (:390-408); a failed step gives
back what it had taken (:838-847).

What is new here, because the reference never splits a prompt and never evicts
(:594-613): every step gives each decoding request its one row first and fills the rest of
the budget with prompt portions, the last one cut to fit, so portions and decoded tokens
share a step.  When pages run out:

1. a prompt portion is cut down to the pages that are free (a request that gets none waits);
2. if a decoding request cannot get the page for its next token, the request that was
   admitted last is preempted: its pages are freed, its tokens (prompt and output so far)
   are kept, and it goes back to the head of the waiting queue to be recomputed;
3. a request that could not fit even with the whole pool to itself is finished with the
   reason ``"cache_full"``; nothing else is disturbed.

The decisions themselves are taken in C++ (the scheduler section of csrc/host_core.cu, which
works on the cache's books directly); this module holds the request and entry types and the
class that keeps the Python ``Request`` objects in step with the records there.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np

from ..cache.manager import CacheManager, RequestCache
from ..sampling.params import SamplingParams


@dataclass(eq=False)            # requests are compared by identity: membership tests must not walk token lists
class Request:
    request_id: Hashable
    prompt: List[int]
    sampling: SamplingParams
    output_ids: List[int] = field(default_factory=list)
    handle: Optional[RequestCache] = None
    finished: bool = False
    finish_reason: Optional[str] = None      # "stop" | "length" | "context" | "cache_full" | "abort"
    cached_tokens: int = 0                   # prompt tokens that were not computed again (prefix reuse)
    preemptions: int = 0
    admitted_at: int = -1
    published_pages: int = 0                 # prompt pages already handed to the prefix tree
    #: tokens that a step has chosen for this request but that have not reached the host yet (0 or 1):
    #: they count as tokens of the request, their values are on the device
    pending: int = 0
    #: the request's record in the C++ scheduler (-1: none), and whether its end has been reported
    slot: int = field(default=-1, repr=False)
    reported: bool = field(default=False, repr=False)

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output_ids) + self.pending

    @property
    def last_token(self) -> int:
        """The last token, or -1 while it is still on the device."""
        if self.pending:
            return -1
        return self.output_ids[-1] if self.output_ids else self.prompt[-1]

    def tokens_from(self, start: int, count: int) -> List[int]:
        """``tokens[start:start + count]`` without building the whole list."""
        n = len(self.prompt)
        if start >= n:
            return self.output_ids[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output_ids[:start + count - n]

    @property
    def computed(self) -> int:
        return self.handle.length if self.handle is not None else 0


@dataclass
class ScheduledEntry:
    request: Request
    tokens: List[int]
    #: True if this portion ends with the request's last known token, so a token is sampled
    samples: bool
    #: True if the entry's one token (-1 here) was chosen by the step before and is still on the device
    from_device: bool = False
    #: the entry as the C++ scheduler gave it: request record, first position, rows, samples, from_device
    record: tuple = (0, 0, 0, 0, 0)


@dataclass
class StepOutput:
    request_id: Hashable
    token_ids: List[int]                     # tokens produced in this step (0 or 1)
    cached_tokens: int
    finished: bool
    finish_reason: Optional[str] = None


@dataclass
class SchedulerConfig:
    max_running_requests: int = 256
    chunked_prefill_size: int = 2048         # token budget of one step
    max_positions: int = 32768               # the model's max_position_embeddings
    default_stop_token_ids: Sequence[int] = ()


REASONS = {0: None, 1: "stop", 2: "length", 3: "context", 4: "cache_full", 5: "abort"}


class Scheduler:
    """The decisions are taken in C++ (csrc/host_core.cu, beside the cache's books); this class keeps
    the Python ``Request`` objects in step with the records there."""

    def __init__(self, cache: CacheManager, config: SchedulerConfig):
        if config.chunked_prefill_size <= 0 or config.max_running_requests <= 0:
            raise ValueError("the token budget and the running limit must be positive")
        self.cache, self.config = cache, config
        lib = self._lib = cache._lib
        lib.hs_create.restype = ctypes.c_void_p
        lib.hs_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_void_p, ctypes.c_int]
        lib.hs_destroy.argtypes = [ctypes.c_void_p]
        lib.hs_set_tree.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        for name in ("hs_add", "hs_forget", "hs_has_work", "hs_schedule", "hs_entries", "hs_entry_tokens", "hs_process",
                     "hs_step_failed", "hs_abort", "hs_release", "hs_mark_pending", "hs_state", "hs_outputs", "hs_queue",
                     "hs_handle_events", "hs_stats", "hs_force_running", "hs_touched"):
            getattr(lib, name).restype = ctypes.c_int
        stops = np.ascontiguousarray(list(config.default_stop_token_ids) or [0], dtype=np.int32)
        pointer = lib.hs_create(cache._pointer, None, int(config.max_running_requests), int(config.chunked_prefill_size),
                                int(config.max_positions), ctypes.c_void_p(stops.ctypes.data),
                                len(config.default_stop_token_ids))
        if not pointer:
            raise ValueError("the scheduler could not be made")
        self._pointer = ctypes.c_void_p(pointer)
        self._requests: Dict[int, Request] = {}             # record in the C++ scheduler -> request
        self._by_handle: Dict[int, Request] = {}            # request of the cache books -> request
        self._state = np.zeros(16, dtype=np.int32)
        self._ended: set = set()                            # finished and reported, record not yet given back
        self._tree = None

    def __del__(self):
        try:
            if getattr(self, "_pointer", None):
                self._lib.hs_destroy(self._pointer)
        except Exception:
            pass

    # ------------------------------------------------------------------ keeping both sides in step
    def _use_tree(self) -> None:
        tree = self.cache.prefix_tree
        if tree is not self._tree:
            self._lib.hs_set_tree(self._pointer, tree._pointer if tree is not None else None)
            self._tree = tree

    def _sync(self, request: Request) -> None:
        state = self._state
        self._lib.hs_state(self._pointer, request.slot, ctypes.c_void_p(state.ctypes.data))
        request.finished = bool(state[1])
        request.finish_reason = REASONS[int(state[2])]
        request.cached_tokens, request.preemptions = int(state[3]), int(state[4])
        request.published_pages, request.pending = int(state[5]), int(state[6])
        request.admitted_at = int(state[9])
        have, total = len(request.output_ids), int(state[7])
        if total > have:
            fresh = np.empty(total - have, dtype=np.int32)
            self._lib.hs_outputs(self._pointer, request.slot, have, ctypes.c_void_p(fresh.ctypes.data), len(fresh))
            request.output_ids.extend(fresh.tolist())

    def _handle_events(self) -> None:
        """Cache requests that the C++ side opened or closed get (or lose) their Python handles."""
        capacity = 3 * 64
        while True:
            out = np.empty(capacity, dtype=np.int32)
            count = self._lib.hs_handle_events(self._pointer, ctypes.c_void_p(out.ctypes.data), capacity)
            if count >= 0:
                break
            capacity *= 4
        for kind, handle_index, slot in out[:3 * count].reshape(-1, 3).tolist():
            if kind == 1:
                request = self._requests[slot]
                request.handle = self.cache.attach(request.request_id, handle_index)
                self._by_handle[handle_index] = request
            else:
                request = self._by_handle.pop(handle_index, None)
                if request is not None and request.handle is not None:
                    self.cache.detach(request.handle)
                    request.handle = None

    # ------------------------------------------------------------------ requests
    def add_request(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        if any(r.request_id == request.request_id and not r.finished for r in self._requests.values()):
            raise ValueError(f"request {request.request_id!r} is queued already")
        prompt = np.ascontiguousarray(request.prompt, dtype=np.int32)
        stops = np.ascontiguousarray(list(request.sampling.stop_token_ids) or [0], dtype=np.int32)
        slot = self._lib.hs_add(self._pointer, ctypes.c_void_p(prompt.ctypes.data), len(prompt),
                                int(min(request.sampling.max_new_tokens, 1 << 30)), ctypes.c_void_p(stops.ctypes.data),
                                len(request.sampling.stop_token_ids), int(bool(request.sampling.ignore_eos)))
        if slot < 0:
            raise ValueError(self._lib.srb_last_error().decode())
        stale = self._requests.get(slot)
        if stale is not None:
            stale.slot = -1
        request.slot = slot
        self._requests[slot] = request

    def _forget_finished(self) -> None:
        """Records of finished requests may be used again (their Python objects keep what they hold)."""
        for slot in list(self._ended):
            request = self._requests[slot]
            self._sync(request)
            if request.reported and request.pending == 0:    # no step in flight still names the record
                self._lib.hs_forget(self._pointer, slot)
                del self._requests[slot]
                self._ended.discard(slot)
                request.slot = -1

    def abort(self, request_id: Hashable) -> bool:
        for request in list(self._requests.values()):
            if request.request_id == request_id and not request.finished:
                done = self._lib.hs_abort(self._pointer, request.slot) == 1
                self._handle_events()
                self._sync_touched()
                self._sync(request)
                return done
        return False

    def abort_all(self) -> int:
        ids = [r.request_id for r in self._requests.values() if not r.finished]
        return sum(self.abort(i) for i in ids)

    @property
    def has_work(self) -> bool:
        return bool(self._lib.hs_has_work(self._pointer))

    def _queue(self, which: int) -> List[Request]:
        out = np.empty(len(self._requests) + 1, dtype=np.int32)
        count = self._lib.hs_queue(self._pointer, which, ctypes.c_void_p(out.ctypes.data), len(out))
        return [self._requests[slot] for slot in out[:count].tolist()]

    @property
    def waiting(self) -> List[Request]:
        return self._queue(0)

    @property
    def running(self) -> List[Request]:
        return self._queue(1)

    @property
    def stats(self) -> Dict[str, int]:
        out = np.zeros(4, dtype=np.int64)
        self._lib.hs_stats(self._pointer, ctypes.c_void_p(out.ctypes.data))
        return {"steps": int(out[0]), "preemptions": int(out[1]), "failed_cache_full": int(out[2]),
                "scheduled_tokens": int(out[3])}

    def release(self, request: Request) -> None:
        """Takes a running request out of the scheduler's hands; the caller now owns its cache handle."""
        if self._lib.hs_release(self._pointer, request.slot) < 0:
            raise RuntimeError(self._lib.srb_last_error().decode())
        self._by_handle.pop(request.handle.index, None)

    def mark_pending(self, request: Request, delta: int = 1) -> None:
        """A token was chosen for the request on the device and has not reached the host yet (+1), or
        it has (-1, which ``process_outputs`` does by itself)."""
        request.pending = self._lib.hs_mark_pending(self._pointer, request.slot, int(delta))

    def _force_running(self, request: Request, handle: RequestCache, admitted_at: int) -> None:
        """For tests that build a state by hand: a waiting request becomes a running one on ``handle``."""
        if self._lib.hs_force_running(self._pointer, request.slot, handle.index, int(admitted_at)) < 0:
            raise RuntimeError(self._lib.srb_last_error().decode())
        request.handle, request.admitted_at = handle, admitted_at
        self._by_handle[handle.index] = request

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self, ahead: bool = False) -> List[ScheduledEntry]:
        """Chooses the rows of the next step and reserves their pages.

        ``ahead``: the step before has not reported its tokens yet (requests have ``pending``
        tokens).  The caller has made sure that every running request can get a page, so nothing
        is preempted; a step with nothing to do is then no deadlock, only a wait for those tokens."""
        self._use_tree()
        count = self._lib.hs_schedule(self._pointer, int(ahead))
        if count < 0:
            raise RuntimeError(self._lib.srb_last_error().decode())
        self._handle_events()
        table = np.empty((max(count, 1), 5), dtype=np.int32)
        self._lib.hs_entries(self._pointer, ctypes.c_void_p(table.ctypes.data))
        total = int(table[:count, 2].sum()) if count else 0
        tokens = np.empty(max(total, 1), dtype=np.int32)
        if self._lib.hs_entry_tokens(self._pointer, ctypes.c_void_p(tokens.ctypes.data), len(tokens)) < 0:
            raise RuntimeError(self._lib.srb_last_error().decode())
        entries: List[ScheduledEntry] = []
        at = 0
        for slot, start, rows, samples, from_device in table[:count].tolist():
            request = self._requests[slot]
            entries.append(ScheduledEntry(request, tokens[at:at + rows].tolist(), bool(samples), bool(from_device),
                                          record=(slot, start, rows, samples, from_device)))
            at += rows
        self._sync_touched()          # entries alone change nothing that a Request shows
        return entries

    def _sync_touched(self) -> None:
        """Whoever was admitted, preempted or finished since the last call shows it."""
        out = np.empty(len(self._requests) + 1, dtype=np.int32)
        count = self._lib.hs_touched(self._pointer, ctypes.c_void_p(out.ctypes.data), len(out))
        for slot in out[:max(count, 0)].tolist():
            request = self._requests.get(slot)
            if request is not None:
                self._sync(request)

    def _is_decoding(self, request: Request) -> bool:
        if request.slot < 0:
            return False
        self._lib.hs_state(self._pointer, request.slot, ctypes.c_void_p(self._state.ctypes.data))
        return bool(self._state[8])

    # ------------------------------------------------------------------ after the step
    def process_outputs(self, entries: Sequence[ScheduledEntry], sampled: Sequence[int]) -> List[StepOutput]:
        """``sampled``: one token per entry with ``samples`` set, in order.  The runner has
        committed the rows already."""
        self._use_tree()
        records = np.ascontiguousarray([e.record for e in entries] or [[0] * 5], dtype=np.int32)
        picks = np.ascontiguousarray(list(sampled) or [0], dtype=np.int32)
        out = np.empty((len(entries) + len(self._requests) + 1, 5), dtype=np.int32)
        count = self._lib.hs_process(self._pointer, ctypes.c_void_p(records.ctypes.data), len(entries),
                                     ctypes.c_void_p(picks.ctypes.data), len(sampled), ctypes.c_void_p(out.ctypes.data),
                                     len(out))
        if count < 0:
            raise RuntimeError(self._lib.srb_last_error().decode())
        self._handle_events()
        self._sync_touched()
        for entry in entries:
            if entry.samples and entry.request.pending:
                entry.request.pending -= 1               # the token has arrived (or its row was in vain)
        outputs: List[StepOutput] = []
        for slot, token, cached, finished, reason in out[:count].tolist():
            request = self._requests[slot]
            if token >= 0 and not finished:
                request.output_ids.append(token)         # a request that ended was brought up to date above
            request.cached_tokens = cached
            if finished:
                request.reported = True
                self._ended.add(slot)
            outputs.append(StepOutput(request.request_id, [token] if token >= 0 else [], cached, bool(finished),
                                      REASONS[reason]))
        self._forget_finished()
        return outputs

    def step_failed(self, entries: Sequence[ScheduledEntry]) -> None:
        """The step raised: every request of the batch is failed and gives its pages back."""
        records = np.ascontiguousarray([e.record for e in entries] or [[0] * 5], dtype=np.int32)
        self._lib.hs_step_failed(self._pointer, ctypes.c_void_p(records.ctypes.data), len(entries))
        self._handle_events()
        self._sync_touched()
        for entry in entries:
            self._sync(entry.request)
