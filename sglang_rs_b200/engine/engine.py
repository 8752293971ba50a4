"""The Python entry point: ``Engine(model_path=...).generate(input_ids, sampling_params)``.

Request lifecycle as in the reference's engine (crates/sglang-srt/src/engine.rs:275-352):
enqueue, run steps until every request has finished, collect ``output_ids``,
``cached_tokens`` and ``finished`` per request (crates/sglang-srt/src/types.rs:71-78).  Here
every step may carry prompt portions and decoded tokens together, and new requests may
join between any two steps (``add_request`` + ``step``).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from typing import Any, Callable, Dict, Hashable, List, Mapping, Optional, Sequence, Union

import torch

from .. import ops
from ..cache.manager import CacheManager
from ..sampling import RequestRandom, Sampler, SamplingParams
from ..weights import load_model, parse_dtype
from .metrics import EngineMetrics
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduler, SchedulerConfig, StepOutput


def kv_bytes_per_token(model, dtype: torch.dtype) -> int:
    from ..parts.base import PagedKV
    width = sum(2 * need.num_kv_heads * need.head_dim for need in model.cache_needs() if isinstance(need, PagedKV))
    return width * (4 if dtype == torch.float32 else 2)


@dataclass
class _StepInFlight:
    """A step that runs on the GPU while the host goes on: its rows, the ids it chose (on the
    device), and the pinned copy of ids and error word that the event says is complete."""
    entries: list
    picked: torch.Tensor
    host: torch.Tensor                       # pinned int32: picked ids, then the error word
    done: torch.cuda.Event


class Engine:
    def __init__(self, model_path: Optional[str] = None, *, random_weights: bool = False, seed: int = 0,
                 dtype: str = "bfloat16", device: str = "cuda", page_size: int = 16,
                 max_total_tokens: Optional[int] = None, mem_fraction_static: float = 0.85,
                 max_running_requests: int = 256, chunked_prefill_size: int = 2048,
                 config: Optional[Mapping[str, Any]] = None, stop_token_ids: Optional[Sequence[int]] = None,
                 disable_cuda_graph: bool = False, disable_radix_cache: bool = False,
                 disable_overlap_schedule: bool = False):
        """Option names follow the reference's server arguments where it has them
        (crates/sglang-srt/src/cli.rs:15-79: ``model_path``, ``device``, ``page_size``,
        ``max_total_tokens``, ``mem_fraction_static``, ``max_running_requests``,
        ``chunked_prefill_size``, ``disable_cuda_graph``, ``disable_radix_cache``; ``disable_overlap_schedule``
        has the name that SGLang gives it).  ``config`` may stand in for the folder's config.json
        together with ``random_weights``."""
        if not str(device).startswith("cuda"):
            raise ValueError(f"device {device!r}: this engine runs on CUDA only and never falls back to the host")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible; this engine has no host path")
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        ops.require_supported_device(self.device)            # before any weight is read
        self.disable_overlap_schedule = disable_overlap_schedule
        self.model = load_model(model_path, device=self.device, dtype=self.dtype, random_weights=random_weights,
                                seed=seed, config=config)
        if max_total_tokens is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            per_token = max(kv_bytes_per_token(self.model, self.dtype), 1)
            # what the step function takes beside the pool, at its largest: the split scratch of captured and of
            # uncaptured steps, the logits that captured steps keep, cuBLAS's workspace
            from .graphs import DecodeGraphs
            from .runner import StepPlanner
            beside = 4 * (StepPlanner.SCRATCH_LIMIT + 2 * DecodeGraphs.SCRATCH_FLOATS) + (64 << 20)
            if not disable_cuda_graph:
                beside += DecodeGraphs.MAX_LOGIT_BYTES
            max_total_tokens = int(max(free - beside, 0) * mem_fraction_static) // per_token
            max_total_tokens = max(page_size, min(max_total_tokens, max_running_requests * self.model.max_positions))
        self.cache = CacheManager(self.model.cache_needs(), page_size=page_size, max_tokens=max_total_tokens,
                                  max_requests=max_running_requests, device=self.device, dtype=self.dtype)
        if not disable_radix_cache and self.cache.prefix_reuse_possible():
            self.cache.enable_prefix_reuse()
        self.runner = ModelRunner(self.model, self.cache, use_cuda_graphs=not disable_cuda_graph)
        stops = tuple(stop_token_ids) if stop_token_ids is not None else tuple(self.model.eos_token_ids)
        self.scheduler = Scheduler(self.cache, SchedulerConfig(
            max_running_requests=max_running_requests, chunked_prefill_size=chunked_prefill_size,
            max_positions=self.model.max_positions, default_stop_token_ids=stops))
        self.sampler = Sampler(self.device, self.model.vocab_size)
        self._randoms: Dict[Hashable, RequestRandom] = {}
        self._requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()
        self._in_flight: Optional[_StepInFlight] = None
        #: totals over the requests (the reference's serving counters); ``metrics.render()`` gives them as text
        self.metrics = EngineMetrics()

    # ------------------------------------------------------------------ low level
    def add_request(self, input_ids: Sequence[int], sampling_params: Union[SamplingParams, Mapping, None] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        ids = [int(t) for t in input_ids]
        for token in ids:
            if not 0 <= token < self.model.vocab_size:
                raise ValueError(f"token id {token} is outside the vocabulary of {self.model.vocab_size}")
        if len(ids) >= self.model.max_positions:
            raise ValueError(f"a prompt of {len(ids)} tokens leaves no room under max_position_embeddings "
                             f"{self.model.max_positions}")
        if request_id is None:
            request_id = f"req-{next(self._ids)}"
        request = Request(request_id, ids, params)
        self.scheduler.add_request(request)
        self._requests[request_id] = request
        self.metrics.arrived(request_id, len(ids))
        self._randoms[request_id] = RequestRandom(request_id, params.seed)
        if params.has_penalties:
            self.sampler.seen.open(request_id, ids)          # the prompt's tokens count as seen
        return request_id

    def step(self, overlap: bool = False) -> List[StepOutput]:
        """One scheduling decision, one model step, one token for every request whose
        portion reached its last token.

        ``overlap``: the step is launched and the call returns what the step *before* produced;
        the host's work for the next step (scheduling, flattening, reading the tokens) then runs
        while the GPU computes.  Tokens of requests that decode go from one step to the next on the
        device.  A request that ends on a stop token has then one more row computed in vain, which
        is dropped.  Call :meth:`drain` (or keep stepping) for the last step's outputs."""
        if overlap:
            return self._step_overlapped()
        outputs = self.drain()
        entries = self.scheduler.schedule()
        if not entries:
            fresh = self.scheduler.process_outputs([], [])
            self._forget_finished(fresh)
            return outputs + fresh
        step_entries = [StepEntry(e.request.handle, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                        for e in entries]
        try:
            logits = self.runner.step(step_entries)
            sampled: List[int] = []
            if logits is not None:
                sampling = [e.request for e in entries if e.samples]
                sampled = self.sampler.sample(
                    logits, [r.sampling for r in sampling], [self._randoms[r.request_id] for r in sampling],
                    [r.request_id for r in sampling])
            self.runner.check_device_errors()
        except Exception:
            self.scheduler.step_failed(entries)
            raise
        fresh = self.scheduler.process_outputs(entries, sampled)
        self._forget_finished(fresh)
        return outputs + fresh

    def _forget_finished(self, outputs: Sequence[StepOutput]) -> None:
        for output in outputs:
            self.metrics.produced(output.request_id, len(output.token_ids), output.finished,
                                  failed=output.finish_reason in ("abort", "cache_full"),
                                  cached_tokens=output.cached_tokens if output.finished else 0)
            if output.finished and self._randoms.pop(output.request_id, None) is not None:
                self.sampler.seen.close(output.request_id)

    # ------------------------------------------------------------------ steps that overlap the host's work
    def _step_overlapped(self) -> List[StepOutput]:
        before = self._in_flight
        launched = None
        if before is not None and self._may_run_ahead():
            launched = self._launch(before)                  # the GPU has its next step before this one is read
        try:
            outputs = self.drain()
        except Exception:
            # the step before failed on the device: the step that ran ahead of it was computed from its
            # tokens, so its requests fail with it (and give their pages back) instead of staying
            # running with a token that never arrives
            if launched is not None:
                self.scheduler.step_failed(launched.entries)
            raise
        if launched is None:
            launched = self._launch(None)
        self._in_flight = launched
        return outputs

    def _may_run_ahead(self) -> bool:
        """The next step can be chosen before the tokens of the one in flight are known: sampling
        needs no token on the host (the counts for penalties live on the device), so what is left to
        ask is whether every running request can get a page without preemption."""
        return self.cache.can_take(len(self.scheduler.running))

    def _launch(self, before: Optional[_StepInFlight]) -> Optional[_StepInFlight]:
        entries = self.scheduler.schedule(ahead=before is not None)
        if not entries:
            return None
        sampling = [e.request for e in entries if e.samples]
        source_row = {}
        if before is not None:
            rows = [e.request for e in before.entries if e.samples]
            source_row = {id(r): i for i, r in enumerate(rows)}
        step_entries = [StepEntry(e.request.handle, [0] if e.from_device else e.tokens,
                                  [len(e.tokens) - 1] if e.samples else [],
                                  token_from=source_row[id(e.request)] if e.from_device else -1) for e in entries]
        try:
            logits = self.runner.step(step_entries, before.picked if before is not None else None)
            if logits is None:
                # nothing to sample: the step is finished here
                self.runner.check_device_errors()
                picked = torch.zeros(1, dtype=torch.int32).pin_memory()
                done = torch.cuda.Event()
                done.record()
                return _StepInFlight(entries, picked[:0].to(self.device, non_blocking=True), picked, done)
            picked = self.sampler.pick_on_device(logits, [r.sampling for r in sampling],
                                                 [self._randoms[r.request_id] for r in sampling],
                                                 [r.request_id for r in sampling])
            host = torch.empty(picked.numel() + 1, dtype=torch.int32, pin_memory=True)
            host[:-1].copy_(picked, non_blocking=True)
            host[-1:].copy_(self.runner.error_word, non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        except Exception:
            self.scheduler.step_failed(entries)
            raise
        for request in sampling:
            self.scheduler.mark_pending(request)
        return _StepInFlight(entries, picked, host, done)

    def drain(self) -> List[StepOutput]:
        """Outputs of the step in flight, if there is one (waits for it)."""
        flight, self._in_flight = self._in_flight, None
        if flight is None:
            return []
        flight.done.synchronize()
        values = flight.host.tolist()
        try:
            self.runner.raise_on_error_bits(values[-1])
        except Exception:
            self.scheduler.step_failed(flight.entries)
            raise
        outputs = self.scheduler.process_outputs(flight.entries, values[:-1])
        self._forget_finished(outputs)
        return outputs

    def abort(self, request_id: Hashable) -> bool:
        self.sampler.seen.close(request_id)
        return self.scheduler.abort(request_id)

    def forward_logits(self, record: Mapping):
        """One step record of trace replay (``{"entries": [{"id", "tokens", "want"}], "end": [...]}``) through
        this engine's model, cache and step function; the wanted logits as a host float32 array, or None.
        For tests: the requests of a trace hold pages of the engine's pool until their ``end``, beside the
        scheduler's requests."""
        from .replay import ReplaySession
        if getattr(self, "_replay", None) is None:
            self._replay = ReplaySession.over(self.model, self.cache, self.runner)
        self.drain()
        return self._replay.run(dict(record))

    def flush_cache(self) -> bool:
        """Possible only while nothing is queued or running, as in the reference
        (crates/sglang-srt/src/scheduler.rs:442-454)."""
        if self.scheduler.has_work or self._in_flight is not None:
            return False
        if self.cache.prefix_tree is not None:
            self.cache.prefix_tree.clear()
        return True

    # ------------------------------------------------------------------ the call a user makes
    def generate(self, input_ids: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling_params: Union[Mapping, Sequence[Mapping], None] = None,
                 sink: Optional[Callable[[int, StepOutput], Any]] = None) -> Union[Dict, List[Dict]]:
        """``input_ids``: one prompt or a list of prompts (token ids).  Returns, per prompt,
        ``{"output_ids", "cached_tokens", "finished", "finish_reason"}``.

        ``sink``: called as ``sink(index of the prompt, output)`` for every step's output of every prompt as soon
        as the step's tokens have reached the host (tokens stream out while generation goes on).  A sink that
        returns ``False`` ends that request: it is aborted, its pages are given back, and what it had produced
        stays in its result (the reference's stream sink has this rule, crates/sglang-srt/src/engine.rs:294-297)."""
        single = len(input_ids) > 0 and not isinstance(input_ids[0], (list, tuple))
        prompts = [input_ids] if single else list(input_ids)
        if isinstance(sampling_params, (list, tuple)):
            if len(sampling_params) != len(prompts):
                raise ValueError("one sampling_params per prompt, or one for all")
            params = list(sampling_params)
        else:
            params = [sampling_params] * len(prompts)
        ids = [self.add_request(prompt, p) for prompt, p in zip(prompts, params)]
        index_of = {request_id: index for index, request_id in enumerate(ids)}
        while self.scheduler.has_work or self._in_flight is not None:
            outputs = self.step(overlap=not self.disable_overlap_schedule)
            if sink is None:
                continue
            for output in outputs:
                index = index_of.get(output.request_id)
                if index is not None and sink(index, output) is False and not output.finished:
                    self.abort(output.request_id)
        results = []
        for request_id in ids:
            request = self._requests.pop(request_id)
            results.append({"output_ids": list(request.output_ids), "cached_tokens": request.cached_tokens,
                            "finished": request.finished, "finish_reason": request.finish_reason})
        return results[0] if single else results
