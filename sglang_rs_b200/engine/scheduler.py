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
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache.manager import CacheManager, OutOfPages, OutOfStateSlots, RequestCache
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


class Scheduler:
    def __init__(self, cache: CacheManager, config: SchedulerConfig):
        if config.chunked_prefill_size <= 0 or config.max_running_requests <= 0:
            raise ValueError("the token budget and the running limit must be positive")
        self.cache, self.config = cache, config
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished_unreported: List[StepOutput] = []
        self._clock = itertools.count()
        self.stats = {"steps": 0, "preemptions": 0, "failed_cache_full": 0, "scheduled_tokens": 0}

    # ------------------------------------------------------------------ requests
    def add_request(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r} has an empty prompt")
        if any(r.request_id == request.request_id for r in itertools.chain(self.waiting, self.running)):
            raise ValueError(f"request {request.request_id!r} is queued already")
        self.waiting.append(request)

    def abort(self, request_id: Hashable) -> bool:
        for queue in (self.waiting, self.running):
            for request in list(queue):
                if request.request_id == request_id:
                    queue.remove(request)
                    self._finish(request, "abort")
                    return True
        return False

    def abort_all(self) -> int:
        ids = [r.request_id for r in itertools.chain(self.waiting, self.running)]
        return sum(self.abort(i) for i in ids)

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self, ahead: bool = False) -> List[ScheduledEntry]:
        """Chooses the rows of the next step and reserves their pages.

        ``ahead``: the step before has not reported its tokens yet (requests have ``pending``
        tokens).  The caller has made sure that every running request can get a page, so nothing
        is preempted; a step with nothing to do is then no deadlock, only a wait for those tokens."""
        while True:
            entries = self._schedule_once()
            if entries or not self.running or ahead:
                break
            # Nothing could move although requests are running: prompts in progress hold all
            # pages between them.  The one admitted last gives its pages up.
            self._preempt(self._youngest_running(), entries)
        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += sum(len(e.tokens) for e in entries)
        return entries

    def _schedule_once(self) -> List[ScheduledEntry]:
        budget = self.config.chunked_prefill_size
        entries: List[ScheduledEntry] = []
        preempted_before = self.stats["preemptions"]

        # 1. every decoding request gets its one row; make room by preemption if needed
        decoding = [r for r in self.running if self._is_decoding(r)]
        for request in decoding:
            if request not in self.running:
                continue                                     # preempted below, earlier in this loop
            if self._ends_whatever_comes(request):
                continue                                     # it finishes when its token arrives
            while True:
                try:
                    self.cache.reserve(request.handle, 1)
                    break
                except OutOfPages:
                    victim = self._youngest_running()
                    if victim is request and len(self.running) == 1:
                        # alone and the pool is full of its own tokens: it can never go on
                        self.running.remove(request)
                        self._finish(request, "cache_full")
                        self.stats["failed_cache_full"] += 1
                        break
                    self._preempt(victim, entries)
                    if victim is request:
                        break
            if request in self.running and not request.finished:
                entries.append(ScheduledEntry(request, [request.last_token], True, from_device=request.pending > 0))
                budget -= 1

        # 2. prompts in progress go on, oldest first; 3. then new requests are admitted
        for request in [r for r in self.running if not self._is_decoding(r)]:
            if budget <= 0:
                break
            if request.pending:
                continue
            if any(e.request is request for e in entries):
                continue
            budget -= self._schedule_portion(request, budget, entries)
        while self.waiting and budget > 0 and len(self.running) < self.config.max_running_requests:
            if self.stats["preemptions"] != preempted_before and self.running:
                break                                        # pages were just taken away: admit nobody this step
            request = self.waiting[0]
            if self._can_never_fit(request):
                self.waiting.popleft()
                self._finish(request, "cache_full")
                self.stats["failed_cache_full"] += 1
                continue
            try:
                request.handle = self.cache.open(request.request_id)
            except OutOfStateSlots:
                break
            tree = self.cache.prefix_tree
            if tree is not None:
                shared = tree.match(request.tokens)
                if shared:
                    self.cache.adopt_prefix(request.handle, ("kv", None), shared)
                    request.published_pages = len(shared)
                    if not request.preemptions:
                        request.cached_tokens = min(request.handle.length, len(request.prompt))
            taken = self._schedule_portion(request, budget, entries)
            if taken == 0:
                self.cache.close(request.handle)             # no page free: it stays at the head
                request.handle = None
                break
            self.waiting.popleft()
            request.admitted_at = next(self._clock)
            self.running.append(request)
            budget -= taken
        return entries

    def _is_decoding(self, request: Request) -> bool:
        return (request.handle is not None and bool(request.output_ids or request.pending)
                and request.computed == request.num_tokens - 1)

    def _ends_whatever_comes(self, request: Request) -> bool:
        """True if the token still on the device is the request's last, whichever it is."""
        return request.pending > 0 and (
            len(request.output_ids) + request.pending >= request.sampling.max_new_tokens
            or request.num_tokens >= self.config.max_positions)

    def _schedule_portion(self, request: Request, budget: int, entries: List[ScheduledEntry]) -> int:
        total = request.num_tokens
        start = request.computed
        count = min(budget, total - start)
        # cut the portion down to the pages that are free
        while count > 0 and not self.cache.can_reserve(request.handle, count):
            free = min(self.cache.free_pages().values(), default=0)
            room = self.cache.capacity(request.handle) - start + free * self.cache.page_size
            count = min(count - 1, max(room, 0))
        if count <= 0:
            return 0
        self.cache.reserve(request.handle, count)
        entries.append(ScheduledEntry(request, request.tokens_from(start, count), start + count == total))
        return count

    def _can_never_fit(self, request: Request) -> bool:
        # prompt (and what was generated before a preemption) plus the token to be sampled next
        need = -(-(request.num_tokens + 1) // self.cache.page_size)
        return any(need > allocator.num_pages for key, allocator in self.cache.allocators.items()
                   if self.cache.windows[key] is None)

    def _youngest_running(self) -> Request:
        return max(self.running, key=lambda r: r.admitted_at)

    def _preempt(self, victim: Request, entries: List[ScheduledEntry]) -> None:
        entries[:] = [e for e in entries if e.request is not victim]
        self.running.remove(victim)
        self.cache.close(victim.handle)
        victim.handle = None
        victim.published_pages = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)

    # ------------------------------------------------------------------ after the step
    def process_outputs(self, entries: Sequence[ScheduledEntry], sampled: Sequence[int]) -> List[StepOutput]:
        """``sampled``: one token per entry with ``samples`` set, in order.  The runner has
        committed the rows already."""
        outputs: List[StepOutput] = list(self.finished_unreported)
        self.finished_unreported.clear()
        picks = iter(sampled)
        tree = self.cache.prefix_tree
        for entry in entries:
            request = entry.request
            if tree is not None and request.handle is not None:
                # full pages of prompt tokens become known as soon as they are computed
                full = min(request.handle.length, len(request.prompt)) // self.cache.page_size
                if full > request.published_pages:
                    tree.insert(request.prompt[:full * self.cache.page_size], request.handle.table(("kv", None))[:full])
                    request.published_pages = full
            if not entry.samples:
                continue
            token = int(next(picks))
            request.pending = max(0, request.pending - 1)
            if request.finished:
                continue                     # it ended (stop token, abort) while this step was already running
            request.output_ids.append(token)
            stops = set(request.sampling.stop_token_ids) | set(self.config.default_stop_token_ids)
            reason = None
            if token in stops and not request.sampling.ignore_eos:
                reason = "stop"
            elif len(request.output_ids) >= request.sampling.max_new_tokens:
                reason = "length"
            elif request.num_tokens >= self.config.max_positions:
                reason = "context"
            if reason:
                self.running.remove(request)
                self._finish(request, reason, report=False)
            outputs.append(StepOutput(request.request_id, [token], request.cached_tokens, request.finished, reason))
        return outputs

    def step_failed(self, entries: Sequence[ScheduledEntry]) -> None:
        """The step raised: every request of the batch is failed and gives its pages back."""
        for entry in entries:
            if entry.request in self.running:
                self.running.remove(entry.request)
                self._finish(entry.request, "abort")

    def _finish(self, request: Request, reason: str, report: bool = True) -> None:
        if request.handle is not None:
            self.cache.close(request.handle)
            request.handle = None
        request.finished, request.finish_reason = True, reason
        if report:
            self.finished_unreported.append(
                StepOutput(request.request_id, [], request.cached_tokens, True, reason))
