"""What the engine counts and logs: per-step records and per-request totals.

``StepStats`` is what :meth:`ModelRunner.step` leaves in ``runner.last_stats`` after every step:
rows, requests, how the rows divide into decoded tokens and prompt portions, pages free, whether the
step ran from a captured graph, the host's time and (once the device has finished it) the device's.
With the environment variable ``SRB_STEP_LOG`` set to a path (or ``stderr``) every step is also
written as one JSON line.  The device time of a step comes from two CUDA events that are read only
after they have completed, so logging never makes the host wait for the GPU.

``EngineMetrics`` holds the totals the reference's serving layer keeps
(crates/sglang-srt/src/serving_metrics.rs:8-54: requests, failed requests, requests in flight,
prompt, generated and cached tokens, time to first token and request duration as sum and count) and
renders them in the same text form.
"""
from __future__ import annotations

import json
import os
import sys
import time
from collections import deque
from dataclasses import asdict, dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, TextIO, Tuple


@dataclass
class StepStats:
    step: int
    rows: int
    requests: int
    decode_rows: int              # entries that bring one token
    prompt_rows: int              # rows of entries that bring more
    wanted: int                   # rows whose logits were asked for
    captured: bool                # replayed from a CUDA graph
    pages_free: Dict[str, int]
    host_ms: float                # wall time of the call on the host (launches are asynchronous)
    device_ms: Optional[float] = None     # between two CUDA events around the step; None until they completed
    kernels: Dict[str, float] = field(default_factory=dict)   # device ms per kernel class (tracing only)

    def to_json(self) -> str:
        return json.dumps(asdict(self), separators=(",", ":"))


def step_log_target() -> Optional[str]:
    return os.environ.get("SRB_STEP_LOG") or None


class StepLog:
    """Collects the steps' records; writes them as JSON lines when a target is given.  Device times are
    filled in from CUDA events once those have completed (checked at later steps and at ``flush``)."""

    def __init__(self, target: Optional[str] = None, keep: int = 4096, time_device: Optional[bool] = None):
        self.target = target
        self.time_device = (target is not None) if time_device is None else bool(time_device)
        self._stream: Optional[TextIO] = None
        self._pending: Deque[Tuple[StepStats, object, object]] = deque()
        self.records: Deque[StepStats] = deque(maxlen=keep)

    def _write(self, stats: StepStats) -> None:
        self.records.append(stats)
        if self.target is None:
            return
        if self._stream is None:
            self._stream = sys.stderr if self.target == "stderr" else open(self.target, "a", encoding="utf-8")
        self._stream.write(stats.to_json() + "\n")
        self._stream.flush()

    def add(self, stats: StepStats, begin=None, end=None) -> None:
        """``begin``, ``end``: CUDA events recorded around the step, or None."""
        if begin is None or end is None:
            self._write(stats)
            return
        self._pending.append((stats, begin, end))
        self.poll()

    def poll(self, wait: bool = False) -> None:
        while self._pending:
            stats, begin, end = self._pending[0]
            if wait:
                end.synchronize()
            elif not end.query():
                break
            stats.device_ms = float(begin.elapsed_time(end))
            self._pending.popleft()
            self._write(stats)

    def flush(self) -> List[StepStats]:
        self.poll(wait=True)
        return list(self.records)


class EngineMetrics:
    """Totals over the engine's requests, in the reference's names."""

    def __init__(self):
        self.requests_total = 0
        self.requests_failed_total = 0
        self.requests_in_flight = 0
        self.prompt_tokens_total = 0
        self.generation_tokens_total = 0
        self.cached_tokens_total = 0
        self.time_to_first_token_seconds_sum = 0.0
        self.time_to_first_token_seconds_count = 0
        self.request_duration_seconds_sum = 0.0
        self.request_duration_seconds_count = 0
        self._started: Dict[Hashable, float] = {}
        self._first: Dict[Hashable, float] = {}
        #: per request (arrival, first token, end), seconds on the host's monotonic clock; kept for callers that
        #: want the distribution and not only the sums
        self.timeline: Dict[Hashable, Tuple[float, Optional[float], Optional[float]]] = {}

    def arrived(self, request_id: Hashable, prompt_tokens: int) -> None:
        now = time.perf_counter()
        self.requests_total += 1
        self.requests_in_flight += 1
        self.prompt_tokens_total += int(prompt_tokens)
        self._started[request_id] = now
        self.timeline[request_id] = (now, None, None)

    def produced(self, request_id: Hashable, tokens: int, finished: bool, failed: bool = False,
                 cached_tokens: int = 0) -> None:
        now = time.perf_counter()
        started = self._started.get(request_id)
        if started is None:
            return
        self.generation_tokens_total += int(tokens)
        arrival, first, _ = self.timeline[request_id]
        if tokens > 0 and request_id not in self._first:
            self._first[request_id] = now
            self.time_to_first_token_seconds_sum += now - started
            self.time_to_first_token_seconds_count += 1
            first = now
        if finished:
            self.requests_in_flight -= 1
            self.requests_failed_total += int(failed)
            self.cached_tokens_total += int(cached_tokens)
            self.request_duration_seconds_sum += now - started
            self.request_duration_seconds_count += 1
            self._started.pop(request_id, None)
            self._first.pop(request_id, None)
            self.timeline[request_id] = (arrival, first, now)
        else:
            self.timeline[request_id] = (arrival, first, None)

    def render(self) -> str:
        """Prometheus text, metric names as in the reference (``sglang_`` prefix)."""
        lines = []
        for name, kind in (("requests_total", "counter"), ("requests_failed_total", "counter"),
                           ("requests_in_flight", "gauge"), ("prompt_tokens_total", "counter"),
                           ("generation_tokens_total", "counter"), ("cached_tokens_total", "counter")):
            lines += [f"# TYPE sglang_{name} {kind}", f"sglang_{name} {getattr(self, name)}"]
        for name in ("time_to_first_token_seconds", "request_duration_seconds"):
            lines += [f"# TYPE sglang_{name} summary", f"sglang_{name}_sum {getattr(self, name + '_sum')}",
                      f"sglang_{name}_count {getattr(self, name + '_count')}"]
        return "\n".join(lines) + "\n"
