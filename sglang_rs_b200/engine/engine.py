"""The Python entry point: ``Engine(model_path=...).generate(input_ids, sampling_params)``.

Request lifecycle as in the reference's engine (crates/sglang-srt/src/engine.rs:275-352):
enqueue, run steps until every request has finished, collect ``output_ids``,
``cached_tokens`` and ``finished`` per request (crates/sglang-srt/src/types.rs:71-78).  Here
every step may carry prompt portions and decoded tokens together, and new requests may
join between any two steps (``add_request`` + ``step``).
"""
from __future__ import annotations

import itertools
from typing import Any, Dict, Hashable, List, Mapping, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..sampling import RequestRandom, Sampler, SamplingParams
from ..weights import load_model, parse_dtype
from .runner import ModelRunner, StepEntry
from .scheduler import Request, Scheduler, SchedulerConfig, StepOutput


def kv_bytes_per_token(model, dtype: torch.dtype) -> int:
    from ..parts.base import PagedKV
    width = sum(2 * need.num_kv_heads * need.head_dim for need in model.cache_needs() if isinstance(need, PagedKV))
    return width * (4 if dtype == torch.float32 else 2)


class Engine:
    def __init__(self, model_path: Optional[str] = None, *, random_weights: bool = False, seed: int = 0,
                 dtype: str = "bfloat16", device: str = "cuda", page_size: int = 16,
                 max_total_tokens: Optional[int] = None, mem_fraction_static: float = 0.85,
                 max_running_requests: int = 256, chunked_prefill_size: int = 2048,
                 config: Optional[Mapping[str, Any]] = None, stop_token_ids: Optional[Sequence[int]] = None,
                 disable_cuda_graph: bool = False, disable_radix_cache: bool = False):
        """Option names follow the reference's server arguments where it has them
        (crates/sglang-srt/src/cli.rs:15-79: ``model_path``, ``device``, ``page_size``,
        ``max_total_tokens``, ``mem_fraction_static``, ``max_running_requests``,
        ``chunked_prefill_size``, ``disable_cuda_graph``, ``disable_radix_cache``).  ``config`` may stand in for the folder's config.json
        together with ``random_weights``."""
        if not str(device).startswith("cuda"):
            raise ValueError(f"device {device!r}: this engine runs on CUDA only and never falls back to the host")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible; this engine has no host path")
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        self.model = load_model(model_path, device=self.device, dtype=self.dtype, random_weights=random_weights,
                                seed=seed, config=config)
        if max_total_tokens is None:
            free, _ = torch.cuda.mem_get_info(self.device)
            per_token = max(kv_bytes_per_token(self.model, self.dtype), 1)
            max_total_tokens = int(free * mem_fraction_static) // per_token
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
        self.sampler = Sampler(self.device)
        self._randoms: Dict[Hashable, RequestRandom] = {}
        self._requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()

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
        self._randoms[request_id] = RequestRandom(request_id, params.seed)
        return request_id

    def step(self) -> List[StepOutput]:
        """One scheduling decision, one model step, one token for every request whose
        portion reached its last token."""
        entries = self.scheduler.schedule()
        if not entries:
            return self.scheduler.process_outputs([], [])
        step_entries = [StepEntry(e.request.handle, e.tokens, [len(e.tokens) - 1] if e.samples else [])
                        for e in entries]
        try:
            logits = self.runner.step(step_entries)
            sampled: List[int] = []
            if logits is not None:
                sampling = [e.request for e in entries if e.samples]
                sampled = self.sampler.sample(
                    logits, [r.sampling for r in sampling], [self._randoms[r.request_id] for r in sampling],
                    [r.tokens if r.sampling.has_penalties else () for r in sampling])
            self.runner.check_device_errors()
        except Exception:
            self.scheduler.step_failed(entries)
            raise
        outputs = self.scheduler.process_outputs(entries, sampled)
        for output in outputs:
            if output.finished:
                self._randoms.pop(output.request_id, None)
        return outputs

    def abort(self, request_id: Hashable) -> bool:
        return self.scheduler.abort(request_id)

    def flush_cache(self) -> bool:
        """Possible only while nothing is queued or running, as in the reference
        (crates/sglang-srt/src/scheduler.rs:442-454)."""
        if self.scheduler.has_work:
            return False
        if self.cache.prefix_tree is not None:
            self.cache.prefix_tree.clear()
        return True

    # ------------------------------------------------------------------ the call a user makes
    def generate(self, input_ids: Union[Sequence[int], Sequence[Sequence[int]]],
                 sampling_params: Union[Mapping, Sequence[Mapping], None] = None) -> Union[Dict, List[Dict]]:
        """``input_ids``: one prompt or a list of prompts (token ids).  Returns, per prompt,
        ``{"output_ids", "cached_tokens", "finished", "finish_reason"}``."""
        single = len(input_ids) > 0 and not isinstance(input_ids[0], (list, tuple))
        prompts = [input_ids] if single else list(input_ids)
        if isinstance(sampling_params, (list, tuple)):
            if len(sampling_params) != len(prompts):
                raise ValueError("one sampling_params per prompt, or one for all")
            params = list(sampling_params)
        else:
            params = [sampling_params] * len(prompts)
        ids = [self.add_request(prompt, p) for prompt, p in zip(prompts, params)]
        while self.scheduler.has_work:
            self.step()
        results = []
        for request_id in ids:
            request = self._requests.pop(request_id)
            results.append({"output_ids": list(request.output_ids), "cached_tokens": request.cached_tokens,
                            "finished": request.finished, "finish_reason": request.finish_reason})
        return results[0] if single else results
