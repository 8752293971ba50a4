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
MAX_LIVE = 4


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens that live requests hold at any time (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE)
    args = parser.parse_args(argv)

    import torch
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no host path", file=sys.stderr)
        return 3
    from ..cache import CacheManager
    from ..weights import load_model, parse_dtype
    from .runner import ModelRunner, StepEntry

    dtype = parse_dtype(args.dtype)
    if dtype == torch.float32:
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    print(f"[trace_run] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    model = load_model(args.model, device="cuda", dtype=dtype)
    # The caller counts each live request's tokens rounded up to 64, a multiple of the page
    # size, so ceil(max_tokens / page_size) pages hold whatever is live at any time.
    cache = CacheManager(model.cache_needs(), page_size=args.page_size, max_tokens=max(args.max_tokens, 1),
                         max_requests=MAX_LIVE,
                         device="cuda", dtype=dtype)
    runner = ModelRunner(model, cache)
    os.makedirs(args.out, exist_ok=True)

    handles = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for item in record.get("entries", []):
            handle = handles.get(item["id"])
            if handle is None:
                handle = handles[item["id"]] = cache.open(item["id"])
            entries.append(StepEntry(handle, item["tokens"], item.get("want", [])))
        logits = runner.step(entries) if entries else None
        if logits is not None:
            host = logits.to(torch.float32).cpu().contiguous().numpy()
            host.astype("<f4", copy=False).tofile(os.path.join(args.out, f"{step}.f32"))
        runner.check_device_errors()
        for request_id in record.get("end", []):
            handle = handles.pop(request_id, None)
            if handle is not None:
                cache.close(handle)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
