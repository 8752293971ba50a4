"""Tracing of the kernels by class, switched on by the environment variable ``SRB_TRACE``.

With ``SRB_TRACE=nvtx`` every call of an op opens an NVTX range named after its class
(``srb/gemm``, ``srb/attention_decode``, ...), which a profiler attached to the process shows.  With
``SRB_TRACE=events`` (or ``1``: both) the call is also bracketed by two CUDA events on the launching
stream; :meth:`KernelTimers.collect` waits for them and returns the device time per class.  A kernel
of a host-bound step is timed from the moment the device reaches it, so gaps in which the device waits
for the host are not counted.  While a stream is being captured into a CUDA graph nothing is
recorded; a replayed graph is timed as a whole by the step's own events.

The reference's profile hook only writes start and stop times (crates/sglang-srt/src/profile.rs:69-101);
this is the per-kernel view that its absence leaves open.
"""
from __future__ import annotations

import functools
import os
from collections import defaultdict
from typing import Dict, List, Optional, Tuple

import torch


class KernelTimers:
    def __init__(self, nvtx: bool = True, events: bool = True):
        self.nvtx, self.events = nvtx, events
        self._depth = 0
        self._open: List[Optional[Tuple[str, torch.cuda.Event]]] = []
        self._pairs: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self.calls: Dict[str, int] = defaultdict(int)

    def begin(self, kind: str) -> None:
        self._depth += 1
        if self._depth > 1:                      # an op called by an op: the outer one is the class that counts
            return
        if torch.cuda.is_current_stream_capturing():
            self._open.append(None)
            return
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"srb/{kind}")
        event = None
        if self.events:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
        self._open.append((kind, event))

    def end(self) -> None:
        self._depth -= 1
        if self._depth > 0:
            return
        opened = self._open.pop()
        if opened is None:
            return
        kind, begin = opened
        self.calls[kind] += 1
        if begin is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pairs.append((kind, begin, end))
        if self.nvtx:
            torch.cuda.nvtx.range_pop()

    def collect(self) -> Dict[str, float]:
        """Device milliseconds per class since the last call (waits for the events)."""
        totals: Dict[str, float] = defaultdict(float)
        for kind, begin, end in self._pairs:
            end.synchronize()
            totals[kind] += float(begin.elapsed_time(end))
        self._pairs.clear()
        return dict(totals)


#: the active timers, or None (the usual case: an op then costs one comparison more)
active: Optional[KernelTimers] = None


def configure(mode: Optional[str]) -> Optional[KernelTimers]:
    """``mode``: None/''/'0' off, 'nvtx', 'events', anything else both."""
    global active
    if not mode or mode in ("0", "off", "false"):
        active = None
    else:
        active = KernelTimers(nvtx=mode != "events", events=mode != "nvtx")
    return active


def traced(kind: str):
    """Decorator of an op: its launches belong to class ``kind``."""
    def wrap(function):
        @functools.wraps(function)
        def inner(*args, **kwargs):
            timers = active
            if timers is None:
                return function(*args, **kwargs)
            timers.begin(kind)
            try:
                return function(*args, **kwargs)
            finally:
                timers.end()
        return inner
    return wrap


configure(os.environ.get("SRB_TRACE"))
