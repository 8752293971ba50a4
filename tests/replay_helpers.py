"""Helpers of the GPU tests: model folders, oracle logits, and ways of cutting requests
into steps.  Traces are lists of the step records that bin/trace_run reads."""
from __future__ import annotations

import os
import random
from typing import Dict, List, Sequence

import numpy as np
import torch

import plain_model as pm

FP32_TOLERANCE = 1e-4      # of the largest |logit| of the oracle
BF16_TOLERANCE = 3e-2      # bfloat16 has 8 bits of mantissa: 8 * 2^-8 of the scale


def make_folder(tmp_path, name: str, config: dict, seed: int, dtype: torch.dtype, sharpen: float = 3.0) -> str:
    """A model folder from the engine's random-weights mode.  The q-norm scales are
    multiplied by ``sharpen`` so that attention is peaked: with flat attention a missing or
    stale key among hundreds would barely move the logits."""
    from sglang_rs_b200.weights import read_model_dir, write_file, write_model_folder
    folder = write_model_folder(str(tmp_path / name), config, seed=seed, dtype=dtype)
    if sharpen != 1.0:
        tensors = {k: v.clone() for k, v in read_model_dir(folder).items()}
        for key in tensors:
            if key.endswith("q_norm.weight"):
                tensors[key] = (tensors[key].float() * sharpen).to(dtype)
        write_file(os.path.join(folder, "model.safetensors"), tensors)
    return folder


def random_requests(config: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(config["vocab_size"]) for _ in range(n)] for i, n in enumerate(lengths)}


def oracle(folder: str, requests: Dict[str, List[int]]) -> Dict[str, np.ndarray]:
    config, weights = pm.load_folder(folder)
    return {rid: pm.plain_forward(config, weights, tokens).numpy() for rid, tokens in requests.items()}


# ------------------------------------------------------------------------------ cuts
def trace_whole(requests):
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def trace_tail_by_one(requests, tail: int = 32):
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for p in range(head, len(toks)):
            steps.append({"entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def trace_portions(requests, sizes=(7, 2, 16, 3, 2, 31, 1, 17, 5, 2, 64, 9)):
    steps, k = [], 0
    for rid, toks in requests.items():
        p = 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}], "end": []})
            p += n
        steps[-1]["end"] = [rid]
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def trace_mixed(requests, seed: int, max_live: int = 4, decode_tail: int = 32,
                portion_sizes=(2, 3, 5, 16, 17, 31, 40), admit: float = 0.6):
    """Up to ``max_live`` live requests; every step mixes portions of some with single
    tokens of others; a request may sit a step out; finished requests end and the next one
    is admitted, so its pages are taken from those just given back."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: Dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < admit):
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for rid in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # left out of this step
            toks, p = requests[rid], live[rid]
            remaining = len(toks) - p
            n = 1 if remaining <= decode_tail else min(rng.choice(portion_sizes), remaining - decode_tail)
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": list(range(n))})
            live[rid] = p + n
            if live[rid] == len(toks):
                end.append(rid)
                del live[rid]
        if entries:
            rng.shuffle(entries)
            steps.append({"entries": entries, "end": end})
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def trace_decode_together(requests, tail: int = 8, prompts_per_step: int = 16):
    """Many requests live at once: their prompts (all but the last ``tail`` tokens) go in steps of
    ``prompts_per_step`` whole prompts, then every step holds one token of every request, so a decode step has
    as many rows as there are requests."""
    steps = []
    names = list(requests)
    for first in range(0, len(names), prompts_per_step):
        steps.append({"entries": [{"id": rid, "tokens": requests[rid][:max(1, len(requests[rid]) - tail)],
                                   "want": [max(1, len(requests[rid]) - tail) - 1]}
                                  for rid in names[first:first + prompts_per_step]], "end": []})
    fed = {rid: max(1, len(requests[rid]) - tail) for rid in names}
    while any(fed[rid] < len(requests[rid]) for rid in names):
        entries, end = [], []
        for rid in names:
            if fed[rid] < len(requests[rid]):
                entries.append({"id": rid, "tokens": [requests[rid][fed[rid]]], "want": [0]})
                fed[rid] += 1
                if fed[rid] == len(requests[rid]):
                    end.append(rid)
        steps.append({"entries": entries, "end": end})
    for i, s in enumerate(steps):
        s["step"] = i
    return steps


def max_tokens_of(trace, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    most = 0
    for step in trace:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return most


def collect(trace, outputs) -> Dict[str, Dict[int, np.ndarray]]:
    """(request, position) -> logits row, from per-step outputs."""
    fed: Dict[str, int] = {}
    rows: Dict[str, Dict[int, np.ndarray]] = {}
    for step, out in zip(trace, outputs):
        k = 0
        for entry in step["entries"]:
            base = fed.get(entry["id"], 0)
            for w in entry["want"]:
                rows.setdefault(entry["id"], {})[base + w] = out[k]
                k += 1
            fed[entry["id"]] = base + len(entry["tokens"])
        assert out is None or k == len(out)
    return rows


def max_live_of(trace) -> int:
    live, most = set(), 0
    for step in trace:
        live |= {entry["id"] for entry in step["entries"]}
        most = max(most, len(live))
        live -= set(step["end"])
    return most


def run_in_process(folder: str, dtype: str, trace, max_tokens=None, page_size: int = 16, graphs: bool = True,
                   radix: bool = False, native_step=None):
    from sglang_rs_b200.engine.replay import ReplaySession
    session = ReplaySession(folder, dtype, max_tokens if max_tokens is not None else max_tokens_of(trace), page_size,
                            use_cuda_graphs=graphs, max_live=max(4, max_live_of(trace)), radix=radix,
                            native_step=native_step)
    outputs = []
    session.page_owners = {}                 # (group, page id) -> requests that held it at some time
    for step in trace:
        outputs.append(session.run(step))
        for rid, handle in session.handles.items():
            for key, table in handle.tables.items():
                for page in table:
                    if page >= 0:
                        session.page_owners.setdefault((key, page), set()).add(rid)
        session.cache.check_invariants()
    held = session.cache.prefix_tree.pages_held if session.cache.prefix_tree is not None else 0
    assert all(a.free_count + held == a.num_pages for a in session.cache.allocators.values()), "pages leaked"
    return collect(trace, outputs), session


def worst_error(rows, expected: Dict[str, np.ndarray]):
    """Largest |difference| over all rows, as a fraction of the largest |logit|, and where."""
    worst, where = 0.0, None
    for rid, by_pos in rows.items():
        scale = float(np.abs(expected[rid]).max())
        for pos, row in sorted(by_pos.items()):
            err = float(np.abs(row.astype(np.float64) - expected[rid][pos]).max()) / scale
            if not np.isfinite(err):
                return float("inf"), (rid, pos)
            if err > worst:
                worst, where = err, (rid, pos)
    return worst, where


def first_bad(rows, expected, tolerance):
    for rid, by_pos in rows.items():
        scale = float(np.abs(expected[rid]).max())
        for pos, row in sorted(by_pos.items()):
            err = float(np.abs(row.astype(np.float64) - expected[rid][pos]).max()) / scale
            if not err <= tolerance:
                return rid, pos, err
    return None
