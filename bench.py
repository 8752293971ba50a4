"""Decode throughput of the engine at the Qwen3-8B shape, random weights, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints one JSON line.  ``value`` is decoded tokens per second of K decode steps at batch 8,
timed on the device with CUDA events; ``e2e`` is the same through the Python entry point
(``Engine.add_request`` / ``Engine.step``: host token ids in through pinned memory, sampled
ids back to the host every step); ``prefill`` is one 2,048-token prompt; ``points`` holds
decode at batch 1 and 64; ``roofline`` divides the bytes a decode step has to read by its
time.  Peaks come from MEASURED_PEAKS.json when present.
"""
from __future__ import annotations

import argparse
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


def qwen3_8b_config(layers: int, max_positions: int = 4096) -> dict:
    """Layer sizes of BASELINE.json configs[2] (Qwen3-8B shape)."""
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
            "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
            "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
            "tie_word_embeddings": False, "max_position_embeddings": max_positions, "hidden_act": "silu",
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


def decode_bytes(model_config: dict, batch: int, context: float) -> float:
    """Bytes one decode step has to read: every weight it uses once, and the cache of the
    live requests (bfloat16)."""
    c = model_config
    q = c["num_attention_heads"] * c["head_dim"]
    kv = c["num_key_value_heads"] * c["head_dim"]
    per_layer = c["hidden_size"] * (q + 2 * kv) + q * c["hidden_size"] + 3 * c["hidden_size"] * c["intermediate_size"]
    weights = (c["num_hidden_layers"] * per_layer + c["vocab_size"] * c["hidden_size"]) * 2
    cache = batch * context * c["num_hidden_layers"] * 2 * kv * 2
    return float(weights + cache)


def prefill_flops(model_config: dict, tokens: int) -> float:
    c = model_config
    q = c["num_attention_heads"] * c["head_dim"]
    kv = c["num_key_value_heads"] * c["head_dim"]
    per_layer = c["hidden_size"] * (q + 2 * kv) + q * c["hidden_size"] + 3 * c["hidden_size"] * c["intermediate_size"]
    gemm = 2.0 * tokens * c["num_hidden_layers"] * per_layer + 2.0 * c["vocab_size"] * c["hidden_size"]   # one logits row
    attention = 2.0 * 2.0 * c["num_hidden_layers"] * c["num_attention_heads"] * c["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--layers", type=int, default=36, help="fewer than 36 only where memory or time needs it")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048, help="tokens each request holds when decoding starts")
    parser.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and the prefill")
    parser.add_argument("--only-prefill", action="store_true",
                        help="run only the prefill of one prompt (for profiling); prints its own short line")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                        help="length of the prompt of --only-prefill (the bench line always uses 2,048)")
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

    import torch
    from sglang_rs_b200 import ops
    from sglang_rs_b200.engine.engine import Engine

    peak, peak_source = peaks()
    config = qwen3_8b_config(args.layers, max(4096, args.context + 2048, args.prefill_tokens + 64))
    torch.manual_seed(0)

    def make_engine(batch: int, steps: int) -> Engine:
        # while later prompts are still computed, earlier requests already decode: leave room for that
        tokens = batch * (args.context + 2 * (steps + warmup) + batch + 64)
        return Engine(config=config, random_weights=True, seed=0, dtype="bfloat16", page_size=16,
                      max_total_tokens=max(tokens, PREFILL_TOKENS + 64, args.prefill_tokens + 64),
                      max_running_requests=max(batch, 1),
                      chunked_prefill_size=2048)

    def prompts(batch: int, length: int):
        g = torch.Generator().manual_seed(batch * 7919 + length)
        return torch.randint(0, config["vocab_size"], (batch, length), generator=g).tolist()

    def decode_run(engine: Engine, batch: int, steps: int, sample_clocks: bool):
        """Prefill ``batch`` requests of ``args.context`` tokens, then time ``steps`` decode
        steps twice: the step function alone on the device, and the whole entry point."""
        from sglang_rs_b200.engine.runner import StepEntry
        ids = [engine.add_request(p, {"max_new_tokens": 1 << 30, "ignore_eos": True}) for p in prompts(batch, args.context)]
        while any(not engine.scheduler._is_decoding(engine._requests[i]) for i in ids):
            engine.step()                                     # portions of prompts until every request decodes
        requests = [engine._requests[i] for i in ids]
        # --- entry point, end to end: every step takes its rows' index arrays from pinned host memory and
        # hands the tokens of the step before back to the host (steps overlap the host's work)
        for _ in range(warmup):
            engine.step(overlap=True)
        engine.drain()
        torch.cuda.synchronize()
        sampler = ClockSampler()
        if sample_clocks:
            sampler.start()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        h2d = engine.runner.planner.last_upload_bytes + (8 * batch if False else 0)
        # --- the step function alone: fixed token ids, logits stay on the device, greedy pick on the device
        handles = [r.handle for r in requests]
        tokens = [[r.tokens[-1]] for r in requests]
        for r, h in zip(requests, handles):                   # the scheduler must not touch them meanwhile
            engine.scheduler.release(r)

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
        print(f"[bench] batch {batch}: step {step_ms:.3f} ms, entry point {e2e_ms:.3f} ms, context {context_mid:.0f}",
              file=sys.stderr, flush=True)
        return {"step_ms": step_ms, "e2e_ms": e2e_ms, "h2d": h2d, "d2h": 4 * batch + 4, "launches": launches,
                "context": context_mid, "clocks": clocks}

    engine = make_engine(max(args.batch, 1), args.steps)
    if args.only_prefill:
        from sglang_rs_b200.engine.runner import StepEntry
        times = []
        length = args.prefill_tokens
        tokens = prompts(1, length)[0]
        for i in range(warmup + args.steps):
            handle = engine.cache.open(f"prefill-{i}")
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            engine.runner.step([StepEntry(handle, tokens, [length - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.cache.close(handle)
            times.append(begin.elapsed_time(end))
        flops = prefill_flops(config, length)
        ms = min(times[warmup:])
        print(json.dumps({"prefill_ms": round(ms, 3), "tokens": length, "layers": args.layers,
                          "frac_of_bf16_peak": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)}))
        return 0
    main_run = decode_run(engine, args.batch, args.steps, sample_clocks=True)
    value = args.batch * 1e3 / main_run["step_ms"]
    need = decode_bytes(config, args.batch, main_run["context"])
    achieved = need / (main_run["step_ms"] * 1e-3) / 1e9
    record = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, random weights)", "value": round(value, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["step_ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) from a seed, uniform random token ids",
        "config": {"model": "Qwen3-8B shape", "layers": args.layers, "layers_of_config": 36, "hidden_size": 4096,
                   "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
                   "vocab_size": 151936, "global_batch": args.batch, "seq_len": args.context,
                   "context_limit": config["max_position_embeddings"], "page_size": 16, "parallelism": "single GPU",
                   "l2": "inputs larger than L2: a step reads all weights"},
        "gpu_launches": main_run["launches"], "clocks": main_run["clocks"],
        "e2e": {"value": round(args.batch * 1e3 / main_run["e2e_ms"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": main_run["h2d"], "d2h_bytes_per_step": main_run["d2h"]},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "of": peak_source},
    }
    if not args.skip_points:
        from sglang_rs_b200.engine.runner import StepEntry
        # prefill of one 2,048-token prompt, timed on the device
        handle = None
        times = []
        for i in range(warmup + 3):
            handle = engine.cache.open(f"prefill-{i}")
            tokens = prompts(1, PREFILL_TOKENS)[0]
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            engine.runner.step([StepEntry(handle, tokens, [PREFILL_TOKENS - 1])])
            end.record()
            torch.cuda.synchronize()
            engine.cache.close(handle)
            if i >= warmup:
                times.append(begin.elapsed_time(end))
        ms = min(times)
        print(f"[bench] prefill {PREFILL_TOKENS} tokens: {ms:.2f} ms", file=sys.stderr, flush=True)
        flops = prefill_flops(config, PREFILL_TOKENS)
        record["prefill"] = {"value": round(PREFILL_TOKENS * 1e3 / ms, 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
                             "frac": round(flops / (ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4),
                             "of": f"{peak_source} bf16_tflops (burst)"}
        points = {}
        one = decode_run(engine, 1, min(args.steps, 32), sample_clocks=False)
        points["decode_b1"] = round(1e3 / one["step_ms"], 2)
        del engine
        torch.cuda.empty_cache()
        big = make_engine(64, min(args.steps, 32))
        many = decode_run(big, 64, min(args.steps, 32), sample_clocks=False)
        points["decode_b64"] = round(64e3 / many["step_ms"], 2)
        record["points"] = points
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
