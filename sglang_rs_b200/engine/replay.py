"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns no forward pass, cache or loader: it opens requests in the
framework's cache manager and calls the same :meth:`ModelRunner.step` that generation
calls.  Steps arrive on standard input, one JSON object a line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted, ``<out>/<step>.f32`` receives them as little-endian
float32 [wanted, vocab], in the order of the entries and of ``want``.  After every step a
line ``done <step>`` is printed and flushed.

With ``--radix`` the session keeps the framework's prefix tree over full pages: a request's
first entry is matched against it and starts on the pages of the longest known prefix (whole
pages only, and never the whole entry: crates/sglang-srt/src/cache.rs:532-540,
crates/sglang-srt/src/scheduler.rs:547-563), and after every step the full pages of the live
requests are made known to the tree.  Wanted rows that lie inside such a prefix are not
computed; their logits are written as NaN.
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
                 device: str = "cuda", use_cuda_graphs: bool = True, max_live: int = DEFAULT_MAX_LIVE,
                 radix: bool = False, native_step=None):
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
        if radix:
            if not self.cache.prefix_reuse_possible():
                raise RuntimeError("this model's cache cannot share prefixes (a window or per-request state)")
            self.cache.enable_prefix_reuse()
        self.runner = ModelRunner(self.model, self.cache, use_cuda_graphs=use_cuda_graphs, native_step=native_step)
        self.handles = {}
        self.history = {}            # request -> every token fed so far (kept only with a prefix tree)
        self.cached_tokens = {}      # request -> tokens its first entry took from the prefix tree

    @classmethod
    def over(cls, model, cache, runner) -> "ReplaySession":
        """A session that drives a model, cache and runner that exist already (an engine's)."""
        session = cls.__new__(cls)
        session.dtype, session.model, session.cache, session.runner, session.handles = runner.dtype, model, cache, runner, {}
        session.history, session.cached_tokens = {}, {}
        return session

    def run(self, record: dict):
        """One step record; returns the wanted logits as a host float32 array, or None."""
        import numpy as np
        from .runner import StepEntry
        tree = self.cache.prefix_tree
        page_size = self.cache.page_size
        entries, layout = [], []
        for item in record.get("entries", []):
            tokens, want = list(item["tokens"]), [int(w) for w in item.get("want", [])]
            handle = self.handles.get(item["id"])
            skipped = 0
            if handle is None:
                handle = self.handles[item["id"]] = self.cache.open(item["id"])
                if tree is not None:
                    pages = tree.match(tokens)             # whole pages, at least one token left to compute
                    if pages:
                        self.cache.adopt_prefix(handle, ("kv", None), pages)
                        skipped = len(pages) * page_size
                    self.cached_tokens[item["id"]] = skipped
            if tree is not None:
                self.history.setdefault(item["id"], []).extend(tokens)
            entries.append(StepEntry(handle, tokens[skipped:], [w - skipped for w in want if w >= skipped]))
            layout.append([w >= skipped for w in want])
        logits = self.runner.step(entries) if entries else None
        host = None
        computed = [flag for flags in layout for flag in flags]
        if logits is not None:
            host = logits.float().cpu().contiguous().numpy()
        if computed and not all(computed):
            full = np.full((len(computed), self.model.vocab_size), np.nan, dtype=np.float32)
            if host is not None:
                full[np.asarray(computed)] = host
            host = full
        self.runner.check_device_errors()
        if tree is not None:
            for entry in entries:                          # pages that are full now become known to the tree
                count = entry.handle.length // page_size
                if count:
                    tokens = self.history[entry.handle.request_id]
                    tree.insert(tokens[:count * page_size], entry.handle.table(("kv", None))[:count])
        for request_id in record.get("end", []):
            handle = self.handles.pop(request_id, None)
            self.history.pop(request_id, None)
            if handle is not None:
                self.cache.close(handle)
        return host


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE)
    parser.add_argument("--max-live", type=int, default=DEFAULT_MAX_LIVE,
                        help="most requests that are live at a time (each holds a slot of per-request state)")
    parser.add_argument("--radix", action="store_true",
                        help="keep the prefix tree: a new request starts on the pages of its longest known prefix")
    return parser


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)

    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    try:
        session = ReplaySession(args.model, args.dtype, args.max_tokens, args.page_size, max_live=args.max_live,
                                radix=args.radix)
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
