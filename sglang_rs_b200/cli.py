"""Command line: ``sglang-rs generate --model-path DIR --device cuda ...``.

Flag names, meanings and defaults follow the reference's argument parser where it has
them (crates/sglang-srt/src/cli.rs:196-462, defaults :651-718): ``--model-path``/``--model``,
``--device``, ``--page-size``, ``--max-total-tokens``, ``--mem-fraction-static``,
``--max-running-requests``, ``--chunked-prefill-size``; ``--flag=value`` is accepted
(:720-723) and unknown flags are kept, not rejected (:575-582).  The reference's only command
starts a server; here the commands are ``generate`` (tokens in, tokens out),
``random-model`` (write a model folder from a config and a seed), ``replay`` and ``bench``.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional


def _ids(text: str) -> List[int]:
    return [int(part) for part in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="sglang-rs")
    commands = parser.add_subparsers(dest="command", required=True)

    gen = commands.add_parser("generate", help="generate tokens for one or more prompts")
    gen.add_argument("--model-path", "--model", dest="model_path", required=True)
    gen.add_argument("--device", default="cuda", help="cuda or cuda:N; there is no host path")
    gen.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    gen.add_argument("--random-weights", action="store_true", help="ignore the folder's weights; draw them from --seed")
    gen.add_argument("--seed", type=int, default=0)
    gen.add_argument("--page-size", type=int, default=16)
    gen.add_argument("--max-total-tokens", "--num-reserved-decode-tokens", dest="max_total_tokens", type=int, default=None,
                     help="tokens the live requests may hold together (the reference counts token slots under the "
                          "second name)")
    gen.add_argument("--mem-fraction-static", type=float, default=0.85)
    gen.add_argument("--max-running-requests", type=int, default=256)
    gen.add_argument("--chunked-prefill-size", "--max-prefill-tokens", dest="chunked_prefill_size", type=int, default=2048,
                     help="token budget of one step: decoded tokens first, prompt portions fill the rest")
    gen.add_argument("--kv-cache-dtype", default="auto", choices=("auto",),
                     help="the cache has the model's dtype; quantized caches are not built")
    gen.add_argument("--disable-cuda-graph", action="store_true")
    gen.add_argument("--disable-radix-cache", action="store_true")
    gen.add_argument("--disable-overlap-schedule", action="store_true",
                     help="read every step's tokens before the next step is launched")
    source = gen.add_mutually_exclusive_group(required=True)
    source.add_argument("--input-ids", action="append", help="comma-separated token ids; repeat for more prompts")
    source.add_argument("--input-ids-file", help="JSON file: a list of token-id lists")
    source.add_argument("--prompt", action="append", help="text, tokenised byte by byte (needs a vocabulary >= 256)")
    gen.add_argument("--max-new-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=None)
    gen.add_argument("--top-p", type=float, default=None)
    gen.add_argument("--top-k", type=int, default=None)
    gen.add_argument("--min-p", type=float, default=None)
    gen.add_argument("--frequency-penalty", type=float, default=None)
    gen.add_argument("--presence-penalty", type=float, default=None)
    gen.add_argument("--repetition-penalty", type=float, default=None)
    gen.add_argument("--sampling-seed", type=int, default=None)
    gen.add_argument("--stop-token-ids", type=_ids, default=None)
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--stream", action="store_true",
                     help="print a JSON line for every step's tokens of every prompt as they reach the host")

    rnd = commands.add_parser("random-model", help="write config.json and model.safetensors from a config and a seed")
    rnd.add_argument("--config", required=True, help="a config.json (or a folder holding one)")
    rnd.add_argument("--out", required=True)
    rnd.add_argument("--seed", type=int, default=0)
    rnd.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))

    commands.add_parser("replay", help="trace replay; same options as bin/trace_run", add_help=False)
    commands.add_parser("bench", help="the benchmark of the repository; same options as bench.py", add_help=False)
    return parser


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    if argv and argv[0] == "bench":
        # bench.py lies beside the package, at the root of the repository
        import os
        import runpy
        script = os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(__file__))), "bench.py")
        if not os.path.exists(script):
            print(f"[sglang-rs] {script} does not exist: the benchmark comes with the repository, not with the package",
                  file=sys.stderr)
            return 2
        saved, sys.argv = sys.argv, [script] + argv[1:]
        try:
            runpy.run_path(script, run_name="__main__")
        except SystemExit as done:
            return int(done.code or 0)
        finally:
            sys.argv = saved
        return 0
    args, extra = build_parser().parse_known_args(argv)
    if extra:
        print(f"[sglang-rs] ignoring unknown arguments: {extra}", file=sys.stderr)

    if args.command == "random-model":
        from .config import RawConfig
        from .weights import parse_dtype, write_model_folder
        document = dict(RawConfig.from_json(args.config).document)
        write_model_folder(args.out, document, args.seed, parse_dtype(args.dtype))
        print(json.dumps({"written": args.out, "seed": args.seed, "dtype": args.dtype}))
        return 0

    from .engine.engine import Engine
    engine = Engine(model_path=args.model_path, random_weights=args.random_weights, seed=args.seed, dtype=args.dtype,
                    device=args.device, page_size=args.page_size, max_total_tokens=args.max_total_tokens,
                    mem_fraction_static=args.mem_fraction_static, max_running_requests=args.max_running_requests,
                    chunked_prefill_size=args.chunked_prefill_size, disable_cuda_graph=args.disable_cuda_graph,
                    disable_radix_cache=args.disable_radix_cache,
                    disable_overlap_schedule=args.disable_overlap_schedule)
    if args.input_ids:
        prompts = [_ids(text) for text in args.input_ids]
    elif args.input_ids_file:
        with open(args.input_ids_file) as handle:
            prompts = json.load(handle)
    else:
        if engine.model.vocab_size < 256:
            raise SystemExit("--prompt needs a vocabulary of at least 256 entries (one per byte)")
        prompts = [list(text.encode("utf-8")) for text in args.prompt]
    sampling = {"max_new_tokens": args.max_new_tokens, "ignore_eos": args.ignore_eos}
    for key in ("temperature", "top_p", "top_k", "min_p", "frequency_penalty", "presence_penalty",
                "repetition_penalty", "stop_token_ids"):
        value = getattr(args, key)
        if value is not None:
            sampling[key] = value
    if args.sampling_seed is not None:
        sampling["seed"] = args.sampling_seed
    sink = None
    if args.stream:
        def sink(index, output):
            print(json.dumps({"index": index, "token_ids": output.token_ids, "finished": output.finished,
                              "finish_reason": output.finish_reason}), flush=True)
    results = engine.generate(prompts, sampling, sink=sink)
    for prompt, result in zip(prompts, results):
        print(json.dumps({"input_ids": prompt, **result}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
