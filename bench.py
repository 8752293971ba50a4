"""Benchmarks of the engine on one B200, random weights, synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape qwen3-8b|qwen3-1.7b|qwen3-32b] [--mode decode|prefill|serve|compare-cublas|kernels|ablate|timeline]

``--mode decode`` (the default) prints the headline JSON line: ``value`` is decoded tokens per second of K
decode steps at batch 8, timed on the device with CUDA events; ``e2e`` is the same through the Python entry
point (``Engine.add_request`` / ``Engine.step``: host token ids in through pinned memory, sampled ids back to
the host every step); ``prefill`` is one 2,048-token prompt; ``points`` holds decode at batch 1 and 64 at both
ends of the context sweep (2,048 and 4,096 tokens), and the host's share of a prefill step and of a mixed
step (decoded rows beside a prompt portion); ``roofline`` divides the bytes a decode step has to read by
its time.  Peaks come from MEASURED_PEAKS.json when present.

``--mode prefill`` (or ``--only-prefill``) times one prompt of ``--prefill-tokens`` tokens alone.
``--mode serve`` runs the continuous-batching workload (128 requests, prompt lengths uniform in [64, 4096],
output lengths uniform in [16, 512], portions of 2,048 tokens) and prints total and generated tokens per
second, the time to the first token and the rows per step.  ``--mode compare-cublas`` times every product
of a layer and the logits product at 1, 8, 64 and 2,048 rows, the engine's own path beside ``torch.mm``
(cuBLAS) of the same shape.  ``--mode kernels`` prints the device time per kernel class of a prefill step
and of a decode step (uncaptured, so that each kernel can be bracketed by events).  ``--mode ablate`` times the
captured decode step with one kind of kernel left out at a time (the step then computes nothing of use): what
each kind costs inside the graph, where kernels overlap their neighbours.  ``--mode timeline`` runs one captured
decode step with kernels built to record when every block starts, stops waiting for the kernels ahead and leaves,
and prints these times launch by launch (use ``--layers 3`` or so); with ``--only-prefill`` the step is one prompt of
``--prefill-tokens`` and the table shows the blocks of the prefill attention tile by tile.

``--shape`` picks the layer sizes (BASELINE.json configs[2], [3], [4]); every mode takes it.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PREFILL_TOKENS = 2048

#: layer sizes of BASELINE.json configs[2], configs[3] and configs[4]
SHAPES = {
    "qwen3-8b": {"num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
                 "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "tie_word_embeddings": False,
                 "context": 4096},
    "qwen3-1.7b": {"num_hidden_layers": 28, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 8,
                   "head_dim": 128, "intermediate_size": 6144, "vocab_size": 151936, "tie_word_embeddings": True,
                   "context": 8192},
    "qwen3-32b": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "num_key_value_heads": 8,
                  "head_dim": 128, "intermediate_size": 25600, "vocab_size": 151936, "tie_word_embeddings": False,
                  "context": 8192},
}


def model_config(shape: str, layers: int | None, max_positions: int) -> dict:
    sizes = dict(SHAPES[shape])
    context = sizes.pop("context")
    if layers is not None:
        sizes["num_hidden_layers"] = layers
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", **sizes, "rope_theta": 1000000.0,
            "rms_norm_eps": 1e-6, "max_position_embeddings": max(context, max_positions), "hidden_act": "silu",
            "attention_bias": False}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            return json.load(handle), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            out, _ = self.process.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
            out, _ = self.process.communicate()
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0])); maxima.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks)}


def layer_products(c: dict) -> dict:
    """(rows of the weight matrix, inner size) of each product of a layer and of the logits."""
    q = c["num_attention_heads"] * c["head_dim"]
    kv = c["num_key_value_heads"] * c["head_dim"]
    return {"qkv": (q + 2 * kv, c["hidden_size"]), "o": (c["hidden_size"], q),
            "gate_up": (2 * c["intermediate_size"], c["hidden_size"]), "down": (c["hidden_size"], c["intermediate_size"]),
            "lm_head": (c["vocab_size"], c["hidden_size"])}


def decode_bytes(c: dict, batch: int, context: float) -> float:
    """Bytes one decode step has to read: every weight it uses once, and the cache of the
    live requests (bfloat16)."""
    products = layer_products(c)
    per_layer = sum(n * k for name, (n, k) in products.items() if name != "lm_head")
    weights = (c["num_hidden_layers"] * per_layer + c["vocab_size"] * c["hidden_size"]) * 2
    cache = batch * context * c["num_hidden_layers"] * 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return float(weights + cache)


def prefill_flops(c: dict, tokens: int) -> float:
    products = layer_products(c)
    per_layer = sum(n * k for name, (n, k) in products.items() if name != "lm_head")
    gemm = 2.0 * tokens * c["num_hidden_layers"] * per_layer + 2.0 * c["vocab_size"] * c["hidden_size"]   # one logits row
    attention = 2.0 * 2.0 * c["num_hidden_layers"] * c["num_attention_heads"] * c["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention


def quantile(values, q: float) -> float:
    ordered = sorted(values)
    return ordered[min(len(ordered) - 1, int(q * len(ordered)))]


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--shape", default="qwen3-8b", choices=sorted(SHAPES))
    parser.add_argument("--mode", default="decode", choices=("decode", "prefill", "serve", "compare-cublas", "kernels", "ablate", "probe-overlap", "timeline"))
    parser.add_argument("--rows", default="1,8,64,2048", help="--mode compare-cublas: the row counts, comma-separated")
    parser.add_argument("--layers", type=int, default=None, help="fewer than the shape has, only where memory or time needs it")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048, help="tokens each request holds when decoding starts")
    parser.add_argument("--skip-points", action="store_true", help="leave out the other batches, contexts and the prefill")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run only the prefill of one prompt (for profiling); prints its own short line")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="length of the prompt of --only-prefill (the bench line always uses 2,048)")
    parser.add_argument("--requests", type=int, default=128, help="--mode serve: number of requests")
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace; this image has no cargo or rustc and no network, so it "
                          "cannot be built or installed offline (pip cannot install a Cargo project)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)

    if args.mode == "timeline":
        # the kernels of a decode step, built with marks that record when each block starts, stops waiting for the
        # kernels ahead and leaves; the variants are files of their own and are loaded in place of the plain builds
        from sglang_rs_b200.csrc.build import compile_library
        for name in TIMELINE_LIBRARIES:
            os.environ[f"SRB_LIBRARY_{name.upper()}"] = compile_library(name, ("SRB_TIMELINE",))

    import torch
    from sglang_rs_b200 import ops
    from sglang_rs_b200.engine.engine import Engine
    from sglang_rs_b200.engine.runner import StepEntry

    peak, peak_source = peaks()
    layers_of_shape = SHAPES[args.shape]["num_hidden_layers"]
    layers = args.layers if args.layers is not None else layers_of_shape
    config = model_config(args.shape, layers, max(4096, args.context + 2048, args.prefill_tokens + 64) + 64)
    torch.manual_seed(0)

    def make_engine(batch: int, steps: int, context: int, extra_tokens: int = 0) -> Engine:
        # while later prompts are still computed, earlier requests already decode: leave room for that
        tokens = batch * (context + 2 * (steps + warmup) + batch + 64) + extra_tokens
        return Engine(config=config, random_weights=True, seed=0, dtype="bfloat16", page_size=16,
                      max_total_tokens=max(tokens, PREFILL_TOKENS + 64, args.prefill_tokens + 64),
                      max_running_requests=max(batch, 1) + 1, chunked_prefill_size=2048)

    def prompts(batch: int, length: int):
        g = torch.Generator().manual_seed(batch * 7919 + length)
        return torch.randint(0, config["vocab_size"], (batch, length), generator=g).tolist()

    def decode_run(engine: Engine, batch: int, steps: int, context: int, sample_clocks: bool, entry_point: bool = True):
        """Prefill ``batch`` requests of ``context`` tokens, then time ``steps`` decode steps twice: the whole
        entry point, and the step function alone on the device."""
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_ms = h2d = None
        sampler = ClockSampler()
        if entry_point:
            ids = [engine.add_request(p, {"max_new_tokens": 1 << 30, "ignore_eos": True}) for p in prompts(batch, context)]
            while any(not engine.scheduler._is_decoding(engine._requests[i]) for i in ids):
                engine.step()                                 # portions of prompts until every request decodes
            requests = [engine._requests[i] for i in ids]
            # --- entry point, end to end: every step takes its rows' index arrays from pinned host memory and
            # hands the tokens of the step before back to the host (steps overlap the host's work)
            for _ in range(warmup):
                engine.step(overlap=True)
            engine.drain()
            torch.cuda.synchronize()
            if sample_clocks:
                sampler.start()
            t0 = time.perf_counter()
            begin.record()
            produced = 0
            for _ in range(steps):
                produced += sum(len(o.token_ids) for o in engine.step(overlap=True))
            produced += sum(len(o.token_ids) for o in engine.drain())
            end.record()
            torch.cuda.synchronize()
            wall = time.perf_counter() - t0
            assert produced == steps * batch, (produced, steps, batch)
            e2e_ms = max(begin.elapsed_time(end), wall * 1e3) / steps
            h2d = engine.runner.planner.last_upload_bytes
            handles = [r.handle for r in requests]
            tokens = [[r.tokens[-1]] for r in requests]
            for r in requests:                                # the scheduler must not touch them meanwhile
                engine.scheduler.release(r)
        else:
            # the prompts go through the step function directly, a portion at a time, so that every request
            # holds exactly ``context`` tokens when the timed steps begin
            names = iter(range(1 << 30))
            handles = [engine.cache.open(f"direct-{batch}-{context}-{next(names)}") for _ in range(batch)]
            for handle, prompt in zip(handles, prompts(batch, context)):
                for first in range(0, context, 2048):
                    engine.runner.step([StepEntry(handle, prompt[first:first + 2048], [])])
            tokens = [[1] for _ in handles]
            if sample_clocks:
                sampler.start()
        # --- the step function alone: fixed token ids, logits stay on the device, greedy pick on the device

        def one_step():
            logits = engine.runner.step([StepEntry(h, t, [0]) for h, t in zip(handles, tokens)])
            return ops.sample(logits, None, None)
        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        launches_before = ops.launch_count
        begin.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sample_clocks else None
        step_ms = begin.elapsed_time(end) / steps
        launches = ops.launch_count - launches_before
        context_mid = sum(h.length for h in handles) / len(handles) - steps / 2
        for h in handles:
            engine.cache.close(h)
        print(f"[bench] batch {batch}: step {step_ms:.3f} ms, entry point "
              f"{'-' if e2e_ms is None else format(e2e_ms, '.3f')} ms, context {context_mid:.0f}", file=sys.stderr, flush=True)
        return {"step_ms": step_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": 4 * batch + 4, "launches": launches,
                "context": context_mid, "clocks": clocks}

    def prefill_run(engine: Engine, length: int, repeats: int):
        """One prompt of ``length`` tokens per step: the device's time (events) and the wall time of steps issued
        back to back (the host's work of step i + 1 runs under the device's work of step i)."""
        tokens = prompts(1, length)[0]
        device = []
        for i in range(warmup + repeats):
            handle = engine.cache.open(f"prefill-{length}-{i}")
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            engine.runner.step([StepEntry(handle, tokens, [length - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.cache.close(handle)
            if i >= warmup:
                device.append(begin.elapsed_time(end))
        handles = [engine.cache.open(f"prefill-wall-{length}-{i}") for i in range(repeats)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for handle in handles:
            engine.runner.step([StepEntry(handle, tokens, [length - 1])])
            engine.cache.close(handle)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3 / repeats
        return min(device), statistics.median(device), wall

    def mixed_run(engine: Engine, batch: int, context: int, portion: int, steps: int):
        """``batch`` decoded rows beside one portion of ``portion`` prompt tokens in every step: device time of a
        step and the wall time per step when steps are issued back to back."""
        ids = [engine.add_request(p, {"max_new_tokens": 1 << 30, "ignore_eos": True}) for p in prompts(batch, context)]
        while any(not engine.scheduler._is_decoding(engine._requests[i]) for i in ids):
            engine.step()
        engine.drain()
        requests = [engine._requests[i] for i in ids]
        handles = [r.handle for r in requests]
        for r in requests:
            engine.scheduler.release(r)
        tokens = [[r.tokens[-1]] for r in requests]
        text = prompts(1, portion)[0]
        counter = iter(range(1 << 30))

        def one_step():
            # the portion is the start of a new prompt every time, so its request stays short
            long = engine.cache.open(f"mixed-portion-{next(counter)}")
            engine.runner.step([StepEntry(h, t, [0]) for h, t in zip(handles, tokens)] + [StepEntry(long, text, [])])
            engine.cache.close(long)
        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        device = []
        for _ in range(3):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            one_step()
            end.record()
            torch.cuda.synchronize()
            device.append(begin.elapsed_time(end))
        t0 = time.perf_counter()
        for _ in range(steps):
            one_step()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3 / steps
        for h in handles:
            engine.cache.close(h)
        return min(device), wall

    shape_note = {"model": f"{args.shape} shape", "layers": layers, "layers_of_config": layers_of_shape,
                  **{k: config[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                            "intermediate_size", "vocab_size")}}

    # ------------------------------------------------------------------ other modes
    if args.mode == "compare-cublas":
        return compare_cublas(args, config, peak, shape_note)
    if args.mode == "serve":
        return serve(args, config, peak, shape_note, warmup)
    if args.mode == "kernels":
        return kernel_classes(args, config, make_engine, prompts, shape_note, warmup)
    if args.mode == "probe-overlap":
        return probe_overlap(args, config)
    if args.mode == "timeline":
        return timeline(args, make_engine, prompts, shape_note)
    if args.mode == "ablate":
        from sglang_rs_b200.ops import records
        engine = make_engine(args.batch, args.steps, args.context)
        steps = min(args.steps, 32)
        times = {}
        for name, bit in [("nothing", 0), *records.SKIP_BITS.items(), ("nothing again", 0)]:
            records.skip = bit
            engine.runner.graphs.captured.clear()                # the choice is made when a step is captured
            try:
                times[name] = decode_run(engine, args.batch, steps, args.context, sample_clocks=False, entry_point=False)["step_ms"]
            finally:
                records.skip = 0
            engine.runner.error_word.zero_()
        whole, again = times.pop("nothing"), times.pop("nothing again")
        per_layer = {name: round((whole - ms) * 1e3 / (1 if name == "head" else layers), 2) for name, ms in times.items()}
        print(json.dumps({"mode": "ablate", "config": {**shape_note, "global_batch": args.batch, "seq_len": args.context},
                          "step_ms": round(whole, 4), "step_ms_measured_again_at_the_end": round(again, 4),
                          "us_per_layer_with_all_kernels": round(whole * 1e3 / layers, 2),
                          "us_saved_per_layer_by_leaving_out": per_layer,
                          "note": "captured decode steps; 'head' is per step, not per layer; a kernel's saving is what it "
                                  "costs beyond what its neighbours hide"}))
        return 0

    short = min(args.steps, 32)
    end_context = SHAPES[args.shape]["context"] if args.shape == "qwen3-8b" else 4096
    late = max(args.context, end_context - (short + warmup) - 8)           # the far end of the context sweep
    engine = make_engine(max(args.batch, 1), args.steps, args.context if args.skip_points else late,
                         extra_tokens=max(4096, args.prefill_tokens))
    if args.only_prefill or args.mode == "prefill":
        best, median, wall = prefill_run(engine, args.prefill_tokens, args.steps)
        flops = prefill_flops(config, args.prefill_tokens)
        print(json.dumps({"prefill_ms": round(best, 3), "median_ms": round(median, 3), "wall_ms_back_to_back": round(wall, 3),
                          "tokens": args.prefill_tokens, "layers": layers,
                          "frac_of_bf16_peak": round(flops / (best * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}))
        return 0
    main_run = decode_run(engine, args.batch, args.steps, args.context, sample_clocks=True)
    value = args.batch * 1e3 / main_run["step_ms"]
    need = decode_bytes(config, args.batch, main_run["context"])
    achieved = need / (main_run["step_ms"] * 1e-3) / 1e9
    record = {
        "metric": f"decode tok/s at batch {args.batch} ({args.shape} shape, random weights)", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["step_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) from a seed, uniform random token ids",
        "config": {**shape_note, "global_batch": args.batch, "seq_len": args.context,
                   "context_limit": config["max_position_embeddings"], "page_size": 16, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: a step reads all weights"},
        "gpu_launches": main_run["launches"], "clocks": main_run["clocks"],
        "e2e": {"value": round(args.batch * 1e3 / main_run["e2e_ms"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "of": peak_source},
    }
    if not args.skip_points:
        best, median, wall = prefill_run(engine, PREFILL_TOKENS, 3)
        print(f"[bench] prefill {PREFILL_TOKENS} tokens: {best:.2f} ms on the device, {wall:.2f} ms a step back to back",
              file=sys.stderr, flush=True)
        flops = prefill_flops(config, PREFILL_TOKENS)
        record["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / best, 1), "tokens": PREFILL_TOKENS, "ms": round(best, 3),
                             "frac": round(flops / (best * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                             "of": f"{peak_source} bf16_tflops (burst)"}
        points = {"prefill_wall_over_device": round(wall / median, 4)}
        mixed_device, mixed_wall = mixed_run(engine, 8, args.context, 256, 16)
        print(f"[bench] mixed step (8 decoded rows + 256 prompt tokens): {mixed_device:.3f} ms on the device, "
              f"{mixed_wall:.3f} ms a step back to back", file=sys.stderr, flush=True)
        points["mixed_b8_p256_ms"] = round(mixed_device, 4)
        points["mixed_wall_over_device"] = round(mixed_wall / mixed_device, 4)
        one = decode_run(engine, 1, short, args.context, sample_clocks=False, entry_point=False)
        points["decode_b1"] = round(1e3 / one["step_ms"], 2)
        far = decode_run(engine, 1, short, late, sample_clocks=False, entry_point=False)
        points[f"decode_b1_ctx{end_context}"] = round(1e3 / far["step_ms"], 2)
        far = decode_run(engine, args.batch, short, late, sample_clocks=False, entry_point=False)
        points[f"decode_b{args.batch}_ctx{end_context}"] = round(args.batch * 1e3 / far["step_ms"], 2)
        points[f"decode_b{args.batch}_ctx{end_context}_hbm_frac"] = round(
            decode_bytes(config, args.batch, far["context"]) / (far["step_ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)
        del engine
        gc.collect()                                          # a model and its records for the step executor refer to each other
        torch.cuda.empty_cache()
        big_batch = 64 if args.shape != "qwen3-32b" else 32
        big = make_engine(big_batch, short, late)
        many = decode_run(big, big_batch, short, args.context, sample_clocks=False, entry_point=False)
        points[f"decode_b{big_batch}"] = round(big_batch * 1e3 / many["step_ms"], 2)
        points[f"decode_b{big_batch}_hbm_frac"] = round(
            decode_bytes(config, big_batch, many["context"]) / (many["step_ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)
        many = decode_run(big, big_batch, short, late, sample_clocks=False, entry_point=False)
        points[f"decode_b{big_batch}_ctx{end_context}"] = round(big_batch * 1e3 / many["step_ms"], 2)
        points[f"decode_b{big_batch}_ctx{end_context}_hbm_frac"] = round(
            decode_bytes(config, big_batch, many["context"]) / (many["step_ms"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)
        record["points"] = points
    print(json.dumps(record))
    return 0


# ---------------------------------------------------------------------------------------- products beside cuBLAS
#: the libraries whose kernels make a decode step of few rows; each has srb_set_timeline when built with SRB_TIMELINE
TIMELINE_LIBRARIES = ("elementwise", "rope_kv", "attention_decode", "gemm_bf16", "attention_prefill_tc")
TIMELINE_KINDS = {1: "add + norm", 2: "product", 3: "rope + page write", 4: "decode attention", 5: "prefill attention"}
TIMELINE_PHASES = ("first block starts", "wait for the kernels ahead returns", "block leaves")


def timeline(args, make_engine, prompts, shape_note) -> int:
    """One captured decode step with kernels that record (time, kernel, phase, SM, block) for every block: prints,
    launch by launch, when the blocks started, when their wait for the kernels ahead returned and when they left.
    The marks cost each block some atomics, so a step is a few per cent longer than without them: read the table
    for the order and the overlap of kernels, not for a step's length."""
    import ctypes

    import numpy as np
    import torch
    from sglang_rs_b200 import ops
    from sglang_rs_b200.csrc.build import load_library
    from sglang_rs_b200.engine.runner import StepEntry

    if args.only_prefill:
        # a prompt of --prefill-tokens in one step: only the tcgen05 attention carries marks among its kernels
        # (phase 1 there: set-up complete); the table below is per tile of 128 rows instead of per launch
        engine = make_engine(1, 16, args.prefill_tokens)
        prompt = prompts(1, args.prefill_tokens)[0]
        turn = iter(range(1 << 30))

        def one_step():
            handle = engine.cache.open(f"timeline-prefill-{next(turn)}")
            engine.runner.step([StepEntry(handle, prompt, [args.prefill_tokens - 1])])
            engine.cache.close(handle)
    else:
        engine = make_engine(args.batch, 16, args.context)
        handles = [engine.cache.open(f"timeline-{i}") for i in range(args.batch)]
        for handle, prompt in zip(handles, prompts(args.batch, args.context)):
            for first in range(0, args.context, 2048):
                engine.runner.step([StepEntry(handle, prompt[first:first + 2048], [])])

        def one_step():
            return ops.sample(engine.runner.step([StepEntry(h, [1], [0]) for h in handles]), None, None)
    for _ in range(3 if args.only_prefill else 6):
        one_step()
    torch.cuda.synchronize()
    records = 1 << 18
    log = torch.zeros(1 + 2 * records, dtype=torch.int64, device="cuda")
    for name in TIMELINE_LIBRARIES:
        if load_library(name).srb_set_timeline(ctypes.c_void_p(log.data_ptr()), ctypes.c_longlong(records)) != 0:
            raise RuntimeError(f"{name}: the timeline buffer was refused")
    one_step()
    torch.cuda.synchronize()
    log.zero_()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    one_step()
    end.record()
    torch.cuda.synchronize()
    for name in TIMELINE_LIBRARIES:
        load_library(name).srb_set_timeline(None, ctypes.c_longlong(0))
    host = log.cpu().numpy()
    count = min(int(host[0]), records)
    when = host[1:1 + 2 * count:2].astype(np.int64)
    tag = host[2:2 + 2 * count:2].astype(np.uint64)
    kind = (tag >> np.uint64(56)).astype(int)
    phase = ((tag >> np.uint64(48)) & np.uint64(0xff)).astype(int)
    when = (when - when.min()) / 1000.0
    if args.only_prefill:
        return prefill_attention_table(args, shape_note, when, tag, kind, phase, count, begin.elapsed_time(end))
    rows = []
    for k in TIMELINE_KINDS:
        for ph in range(len(TIMELINE_PHASES)):
            chosen = np.sort(when[(kind == k) & (phase == ph)])
            if not len(chosen):
                continue
            # the marks of one launch lie close together; a gap of more than 1.2 us starts the next launch
            cuts = [0, *(np.nonzero(np.diff(chosen) > 1.2)[0] + 1).tolist(), len(chosen)]
            for a, b in zip(cuts[:-1], cuts[1:]):
                rows.append((float(chosen[a]), float(chosen[b - 1]), b - a, TIMELINE_KINDS[k], TIMELINE_PHASES[ph]))
    rows.sort()
    print(f"{'first us':>9} {'last us':>9} {'blocks':>6}  kernel, what its blocks did", file=sys.stderr)
    for first, last, blocks, name, what in rows:
        print(f"{first:9.2f} {last:9.2f} {blocks:6d}  {name}: {what}", file=sys.stderr)
    print(json.dumps({"mode": "timeline", "config": {**shape_note, "global_batch": args.batch, "seq_len": args.context},
                      "step_us_with_marks": round(begin.elapsed_time(end) * 1e3, 1), "records": count,
                      "note": "the table is on stderr: per launch and phase the time of the first and the last block's "
                              "mark, in us since the step's first mark"}))
    return 0


def prefill_attention_table(args, shape_note, when, tag, kind, phase, count, step_ms) -> int:
    """The blocks of the last layer's prefill attention, tile by tile (a tile: 128 rows of the prompt against the keys
    before and beside them; the grid holds one block per tile and pair of query heads, longest tiles first): when
    they started, how long they stayed, and which SMs took a second block."""
    import numpy as np
    block = (tag & np.uint64(0xffffffff)).astype(int)
    sm = ((tag >> np.uint64(32)) & np.uint64(0xffff)).astype(int)
    mine = kind == 5
    last = {}                                     # (block, phase) -> (time, sm) of the last layer's launch
    for i in np.argsort(when):
        if mine[i]:
            last[(int(block[i]), int(phase[i]))] = (float(when[i]), int(sm[i]))
    blocks = sorted({b for b, _ in last})
    if not blocks:
        print("no marks of the prefill attention: the step did not run the tcgen05 kernel", file=sys.stderr)
        return 1
    head_blocks = shape_note["num_attention_heads"] // 2 if (shape_note["num_attention_heads"] //
                                                           shape_note["num_key_value_heads"]) % 2 == 0 else shape_note["num_attention_heads"]
    base = min(last[(b, 0)][0] for b in blocks)
    print(f"{'tile':>4} {'blocks':>6} {'start us':>17} {'set-up us':>9} {'stay us':>15} {'leave us':>9}", file=sys.stderr)
    for tile in range((len(blocks) + head_blocks - 1) // head_blocks):
        ids = [b for b in blocks if b // head_blocks == tile]
        start = np.array([last[(b, 0)][0] - base for b in ids])
        ready = np.array([last[(b, 1)][0] - last[(b, 0)][0] for b in ids])
        leave = np.array([last[(b, 2)][0] - base for b in ids])
        print(f"{tile:4d} {len(ids):6d} {start.min():7.1f} ..{start.max():7.1f} {ready.mean():9.1f} "
              f"{(leave - start).min():6.1f} ..{(leave - start).max():6.1f} {leave.max():9.1f}", file=sys.stderr)
    per_sm = {}
    for b in blocks:
        per_sm.setdefault(last[(b, 0)][1], []).append(b)
    print(f"{len(blocks)} blocks on {len(per_sm)} SMs; SMs with two or more blocks: {sum(len(v) > 1 for v in per_sm.values())}",
          file=sys.stderr)
    print(json.dumps({"mode": "timeline", "config": {**shape_note, "prefill_tokens": args.prefill_tokens},
                      "step_ms_with_marks": round(step_ms, 3), "records": count,
                      "attention_us_last_layer": round(max(last[(b, 2)][0] for b in blocks) - base, 1),
                      "note": "the table is on stderr: the last layer's prefill attention, per tile of 128 rows"}))
    return 0


def compare_cublas(args, config, peak, shape_note) -> int:
    """Every product of a layer and the logits product at 1, 8, 64 and 2,048 rows: the path the engine takes
    (``ops.linear`` / ``ops.gated_product``: this package's tcgen05 kernels up to 64 rows and for gate/up of long
    portions, the library elsewhere) beside ``torch.mm`` of the same shape, which is the call the reference's
    engine makes for every projection (crates/sglang-kernel/src/cublas.rs:383-410).  Timed with CUDA events over
    weights that rotate through copies larger than L2 together, so every call streams them from memory."""
    import torch
    from sglang_rs_b200 import ops
    device = torch.device("cuda")
    word = ops.new_error_word(device)
    inner = config["intermediate_size"]
    rows_list = tuple(int(r) for r in args.rows.split(","))
    results = []
    generator = torch.Generator(device=device).manual_seed(args.seed)
    for name, (n, k) in layer_products(config).items():
        copies = max(2, int(300e6 // (n * k * 2)) + 1)                     # more than twice L2 in rotation
        weights = [(torch.randn(n, k, device=device, generator=generator) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for m in rows_list:
            x = (torch.randn(m, k, device=device, generator=generator)).to(torch.bfloat16)

            def own(w):
                if name == "gate_up":
                    return ops.gated_product(x, w, inner, word)
                if name == "lm_head":
                    return ops.linear(x, w, out_dtype=torch.float32, error_word=word)
                return ops.linear(x, w, error_word=word, partial_ok=True)

            def library(w):
                if name == "gate_up":
                    both = torch.mm(x, w.t())
                    out = torch.empty(m, inner, dtype=torch.bfloat16, device=device)
                    ops.gated_mul(both, out)
                    return out
                if name == "lm_head":
                    return torch.mm(x, w.t(), out_dtype=torch.float32)
                return torch.mm(x, w.t())

            def timed(call):
                for i in range(3):
                    call(weights[i % copies])
                torch.cuda.synchronize()
                repeats = 20 if m <= 64 else 10
                replayed = m <= 1024
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if replayed:
                    # some tens of microseconds of kernel each: launched one by one the host would be what is timed
                    # (this package's call goes through Python), so the calls are captured into one graph (as the
                    # engine's decode steps are) and replayed
                    graph = torch.cuda.CUDAGraph()
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side), ops.stream_scope():
                            for i in range(repeats):
                                call(weights[(i + 3) % copies])
                    torch.cuda.current_stream().wait_stream(side)
                    graph.replay()
                    torch.cuda.synchronize()
                    begin.record()
                    graph.replay()
                    end.record()
                else:
                    begin.record()
                    for i in range(repeats):
                        call(weights[(i + 3) % copies])
                    end.record()
                torch.cuda.synchronize()
                return begin.elapsed_time(end) * 1e3 / repeats
            own_us, library_us = timed(own), timed(library)
            entry = {"product": name, "rows": m, "weight": [n, k], "own_us": round(own_us, 2), "cublas_us": round(library_us, 2),
                     "own_over_cublas": round(library_us / own_us, 3)}
            if m >= 256 and name not in ("gate_up", "lm_head"):
                # the CTA-pair kernel on a plain product (the engine leaves these to the library)
                pair_us = timed(lambda w: ops.gemm_bf16_pair(x, w, word, mode="bf16"))
                entry["pair_kernel_us"] = round(pair_us, 2)
                entry["pair_kernel_tflops"] = round(2.0 * m * n * k / (pair_us * 1e-6) / 1e12, 1)
            if m <= 512:
                entry["own_hbm_frac"] = round(n * k * 2 / (own_us * 1e-6) / 1e9 / peak["hbm_gbs"], 3)
                entry["cublas_hbm_frac"] = round(n * k * 2 / (library_us * 1e-6) / 1e9 / peak["hbm_gbs"], 3)
            if m > 64:
                entry["own_tflops"] = round(2.0 * m * n * k / (own_us * 1e-6) / 1e12, 1)
                entry["cublas_tflops"] = round(2.0 * m * n * k / (library_us * 1e-6) / 1e12, 1)
            results.append(entry)
            print(f"[bench] {name:8s} rows {m:5d}: own {own_us:9.2f} us, cuBLAS {library_us:9.2f} us", file=sys.stderr, flush=True)
        del weights
        torch.cuda.empty_cache()
    ops.raise_on_error_word(word)
    print(json.dumps({"mode": "compare-cublas", "config": shape_note, "timing": "CUDA events, weights rotate through copies "
                      "larger than L2; up to 1,024 rows the calls are replayed from one CUDA graph; gate_up includes the activation (own: in the epilogue; cuBLAS: a kernel after it)",
                      "products": results}))
    return 0


# ---------------------------------------------------------------------------------------- do kernels overlap?
def probe_overlap(args, config) -> int:
    """The library's gate/up and down products of ``--prefill-tokens`` rows on one stream and this package's norm
    kernel on another: alone, and together.  (What two halves of a prompt on two streams could hide of the
    memory-bound kernels under the products.)"""
    import torch
    from sglang_rs_b200 import ops
    device = torch.device("cuda")
    rows, hidden, inner = args.prefill_tokens, config["hidden_size"], config["intermediate_size"]
    x = torch.randn(rows, hidden, device=device).bfloat16()
    act = torch.randn(rows, inner, device=device).bfloat16()
    w_gate_up = (torch.randn(2 * inner, hidden, device=device) * 0.02).bfloat16()
    w_down = (torch.randn(hidden, inner, device=device) * 0.02).bfloat16()
    residual, delta = torch.randn(rows, hidden, device=device), torch.randn(rows, hidden, device=device).bfloat16()
    weight, out = torch.ones(hidden, device=device), torch.empty(rows, hidden, device=device, dtype=torch.bfloat16)
    word = ops.new_error_word(device)

    def products():
        for _ in range(10):
            ops.linear(x, w_gate_up, error_word=word)
            ops.linear(act, w_down, error_word=word)

    def norms():
        for _ in range(40):
            ops.add_rmsnorm(residual, delta, weight, 1e-6, out)

    def timed(call):
        call()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        call()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end)
    one, two = torch.cuda.Stream(), torch.cuda.Stream()

    def together():
        current = torch.cuda.current_stream()
        one.wait_stream(current)
        two.wait_stream(current)
        with torch.cuda.stream(one), ops.stream_scope():
            products()
        with torch.cuda.stream(two), ops.stream_scope():
            norms()
        current.wait_stream(one)
        current.wait_stream(two)
    print(json.dumps({"mode": "probe-overlap", "rows": rows, "products_alone_ms": round(timed(products), 3),
                      "norms_alone_ms": round(timed(norms), 3), "together_on_two_streams_ms": round(timed(together), 3),
                      "what": "10 x (gate/up + down) by the library on one stream, 40 add+norm kernels on another"}))
    return 0


# ---------------------------------------------------------------------------------------- continuous batching
def serve(args, config, peak, shape_note, warmup) -> int:
    """BASELINE.json configs[3]: ``--requests`` requests, prompt lengths uniform in [64, 4096], output lengths
    uniform in [16, 512], all queued at the start, portions of 2,048 tokens, through ``Engine.step``."""
    import random

    import torch
    from sglang_rs_b200.engine.engine import Engine
    rng = random.Random(args.seed)
    lengths = [(rng.randint(64, 4096), rng.randint(16, 512)) for _ in range(args.requests)]
    most = max(p + o for p, o in lengths)
    config = dict(config, max_position_embeddings=max(config["max_position_embeddings"], most + 16))
    total_tokens = sum(p + o for p, o in lengths)
    engine = Engine(config=config, random_weights=True, seed=0, dtype="bfloat16", page_size=16,
                    max_total_tokens=total_tokens + 64 * args.requests, max_running_requests=args.requests,
                    chunked_prefill_size=2048, disable_radix_cache=True)
    generator = torch.Generator().manual_seed(args.seed)
    prompts = [torch.randint(0, config["vocab_size"], (p,), generator=generator).tolist() for p, _ in lengths]

    def run_once():
        t0 = time.perf_counter()
        ids = [engine.add_request(prompt, {"max_new_tokens": o, "ignore_eos": True}) for prompt, (_, o) in zip(prompts, lengths)]
        generated = 0
        while engine.scheduler.has_work or engine._in_flight is not None:
            generated += sum(len(o.token_ids) for o in engine.step(overlap=True))
        torch.cuda.synchronize()
        return ids, generated, time.perf_counter() - t0
    # warm-up: the same workload once, so that the graphs of its decode steps are captured and the libraries have
    # settled; the timed run then is the steady state of a server that has seen such requests before
    warm_ids, _, warm_wall = run_once()
    for request_id in warm_ids:
        engine._requests.pop(request_id, None)
    engine.runner.step_log.flush()
    engine.runner.step_log.records.clear()
    steps_before = engine.runner.steps_run
    torch.cuda.synchronize()
    sampler = ClockSampler()
    sampler.start()
    ids, generated, wall = run_once()
    clocks = sampler.stop()
    records = list(engine.runner.step_log.flush())
    first = [engine.metrics.timeline[i][1] - engine.metrics.timeline[i][0] for i in ids]
    done = [engine.metrics.timeline[i][2] - engine.metrics.timeline[i][0] for i in ids]
    assert generated == sum(o for _, o in lengths), (generated, sum(o for _, o in lengths))
    rows = [r.rows for r in records]
    print(json.dumps({
        "mode": "serve", "metric": "continuous batching, tokens/s (prompt + generated) over the whole run",
        "value": round(total_tokens / wall, 1), "unit": "tokens/s", "generated_tokens_per_s": round(generated / wall, 1),
        "wall_s": round(wall, 3), "first_run_wall_s": round(warm_wall, 3), "requests": args.requests, "prompt_tokens": sum(p for p, _ in lengths),
        "generated_tokens": generated,
        "ttft_s": {"mean": round(statistics.mean(first), 4), "p50": round(quantile(first, 0.5), 4),
                   "p99": round(quantile(first, 0.99), 4)},
        "request_s": {"mean": round(statistics.mean(done), 4), "p99": round(quantile(done, 0.99), 4)},
        "steps": engine.runner.steps_run - steps_before,
        "rows_per_step": {"mean": round(statistics.mean(rows), 1), "max": max(rows)},
        "steps_from_graphs": sum(r.captured for r in records), "mixed_steps": sum(bool(r.prompt_rows and r.decode_rows) for r in records),
        "host_ms_per_step": round(statistics.mean(r.host_ms for r in records), 3),
        "preemptions": engine.scheduler.stats.get("preemptions"), "clocks": clocks, "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids, seeded lengths",
        "config": {**shape_note, "chunked_prefill_size": 2048, "page_size": 16, "prompt_len": "U[64,4096]",
                   "output_len": "U[16,512]", "arrival": "all at the start"}}))
    return 0


# ---------------------------------------------------------------------------------------- kernel classes
def kernel_classes(args, config, make_engine, prompts, shape_note, warmup) -> int:
    """Device time per kernel class (CUDA events around every op) of one prefill step of 2,048 tokens and of one
    decode step at ``--batch`` and ``--context``, both uncaptured."""
    import torch
    from sglang_rs_b200.engine.runner import StepEntry
    from sglang_rs_b200.ops import trace
    length = args.prefill_tokens
    engine = make_engine(args.batch, 8, args.context, extra_tokens=max(4096, length + 64))
    engine.runner.graphs = None                              # every kernel launched on its own
    out = {"mode": "kernels", "config": shape_note, "note": "CUDA events around every op of an uncaptured step; "
           "shares, not absolutes: a captured decode step is shorter than the sum"}
    tokens = prompts(1, length)[0]
    out["prefill_tokens"] = length
    handles = [engine.cache.open(f"d{i}") for i in range(args.batch)]
    for handle, prompt in zip(handles, prompts(args.batch, args.context)):
        engine.runner.step([StepEntry(handle, prompt, [])])
    for name in ("prefill", "decode"):
        totals = []
        for i in range(warmup + 3):
            if i == warmup:
                trace.configure("events")
            if name == "prefill":
                handle = engine.cache.open(f"p{i}")
                engine.runner.step([StepEntry(handle, tokens, [length - 1])])
                engine.cache.close(handle)
            else:
                engine.runner.step([StepEntry(h, [1], [0]) for h in handles])
            if i >= warmup:
                totals.append(dict(engine.runner.last_stats.kernels, step_device_ms=engine.runner.step_log.flush()[-1].device_ms))
        trace.configure(None)
        keys = sorted({k for t in totals for k in t})
        out[name] = {k: round(min(t.get(k, 0.0) for t in totals), 4) for k in keys}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
