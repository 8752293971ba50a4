"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns no forward pass, cache or loader: it opens requests in the
framework's cache manager and calls the same :meth:`ModelRunner.step` that generation
calls.  Steps arrive on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted, ``<out>/<step>.f32`` receives them as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After every step a
line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE_SIZE = 16
#: requests that may be live at a time unless ``--max-live`` says otherwise
DEFAULT_MAX_LIVE = 4


class ReplaySession:
    """A model, a cache pool for ``max_tokens`` tokens and the step function, driven by
    step records.  Used by the command line below and by tests."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = PAGE_SIZE,
                 device: str = "cuda", use_cuda_graphs: bool = True, max_live: int = DEFAULT_MAX_LIVE):
        import torch
        from ..cache import CacheManager
        from ..weights import load_model, parse_dtype
        from .runner import ModelRunner
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device; this engine has no host path")
        self.dtype = parse_dtype(dtype)
        self.model = load_model(model_dir, device=device, dtype=self.dtype)
        # The caller counts each live request's tokens rounded up to 64, a multiple of the page
        # size, so ceil(max_tokens / page_size) pages hold whatever is live at any time.
        self.cache = CacheManager(self.model.cache_needs(), page_size=page_size, max_tokens=max(max_tokens, 1),
                                  max_requests=max(int(max_live), 1), device=device, dtype=self.dtype)
        self.runner = ModelRunner(self.model, self.cache, use_cuda_graphs=use_cuda_graphs)
        self.handles = {}

    @classmethod
    def over(cls, model, cache, runner) -> "ReplaySession":
        """A session that drives a model, cache and runner that exist already (an engine's)."""
        session = cls.__new__(cls)
        session.dtype, session.model, session.cache, session.runner, session.handles = runner.dtype, model, cache, runner, {}
        return session

    def run(self, record: dict):
        """One step record; returns the wanted logits as a host float32 array, or None."""
        from .runner import StepEntry
        entries = []
        for item in record.get("entries", []):
            handle = self.handles.get(item["id"])
            if handle is None:
                handle = self.handles[item["id"]] = self.cache.open(item["id"])
            entries.append(StepEntry(handle, item["tokens"], item.get("want", [])))
        logits = self.runner.step(entries) if entries else None
        host = None
        if logits is not None:
            host = logits.float().cpu().contiguous().numpy()
        self.runner.check_device_errors()
        for request_id in record.get("end", []):
            handle = self.handles.pop(request_id, None)
            if handle is not None:
                self.cache.close(handle)
        return host


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE)
    parser.add_argument("--max-live", type=int, default=DEFAULT_MAX_LIVE,
                        help="most requests that are live at a time (each holds a slot of per-request state)")
    args = parser.parse_args(argv)

    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    try:
        session = ReplaySession(args.model, args.dtype, args.max_tokens, args.page_size, max_live=args.max_live)
    except RuntimeError as error:
        print(f"trace_run: {error}", file=sys.stderr)
        return 3
    os.makedirs(args.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = session.run(record)
        if logits is not None:
            logits.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{record['step']}.f32"))
        print(f"done {record['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
