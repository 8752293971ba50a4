"""The command line's option names and their meanings (no GPU): the reference's names where it has them
(crates/sglang-srt/src/cli.rs:196-462), ``--flag=value`` (:720-723), unknown flags kept (:575-582)."""
import pytest

from sglang_rs_b200.cli import build_parser


def parse(*argv):
    return build_parser().parse_known_args(list(argv))


def test_generate_takes_the_reference_names_and_their_aliases():
    args, extra = parse("generate", "--model", "/m", "--input-ids", "1,2,3", "--page-size=8", "--max-running-requests", "7",
                        "--num-reserved-decode-tokens", "4096", "--max-prefill-tokens", "512", "--kv-cache-dtype", "auto",
                        "--disable-radix-cache", "--disable-cuda-graph", "--disable-overlap-schedule",
                        "--mem-fraction-static=0.5", "--not-an-option", "--tp-size", "1")
    assert (args.model_path, args.page_size, args.max_running_requests) == ("/m", 8, 7)
    assert args.max_total_tokens == 4096 and args.chunked_prefill_size == 512 and args.mem_fraction_static == 0.5
    assert args.disable_radix_cache and args.disable_cuda_graph and args.disable_overlap_schedule
    assert extra == ["--not-an-option", "--tp-size", "1"]             # kept for the caller to report, not an error
    args, _ = parse("generate", "--model-path", "/m", "--input-ids", "1", "--max-total-tokens", "99",
                    "--chunked-prefill-size", "64")
    assert (args.max_total_tokens, args.chunked_prefill_size, args.device, args.dtype) == (99, 64, "cuda", "bfloat16")


def test_sampling_options_and_prompts():
    args, _ = parse("generate", "--model-path", "/m", "--input-ids", "5 6", "--input-ids", "7,8", "--temperature", "0.7",
                    "--top-p", "0.9", "--top-k", "40", "--min-p", "0.05", "--repetition-penalty", "1.1",
                    "--presence-penalty", "0.2", "--frequency-penalty", "-0.1", "--sampling-seed", "3",
                    "--stop-token-ids", "9,10", "--ignore-eos", "--max-new-tokens", "4")
    assert args.input_ids == ["5 6", "7,8"] and args.stop_token_ids == [9, 10] and args.ignore_eos and not args.stream
    assert parse("generate", "--model-path", "/m", "--input-ids", "1", "--stream")[0].stream
    assert (args.temperature, args.top_p, args.top_k, args.min_p) == (0.7, 0.9, 40, 0.05)
    assert (args.repetition_penalty, args.presence_penalty, args.frequency_penalty, args.sampling_seed) == (1.1, 0.2, -0.1, 3)
    with pytest.raises(SystemExit):                                   # one source of prompts, not two
        parse("generate", "--model-path", "/m", "--input-ids", "1", "--prompt", "hello")
    with pytest.raises(SystemExit):                                   # a quantized cache is not built
        parse("generate", "--model-path", "/m", "--input-ids", "1", "--kv-cache-dtype", "fp8_e5m2")


def test_random_model_command():
    args, _ = parse("random-model", "--config", "c.json", "--out", "/o", "--seed", "5", "--dtype", "float32")
    assert (args.command, args.config, args.out, args.seed, args.dtype) == ("random-model", "c.json", "/o", 5, "float32")


def test_bench_command_runs_the_benchmark_of_the_repository(capsys):
    from sglang_rs_b200.cli import main
    assert main(["bench", "--impl", "reference"]) == 0
    assert '"impl": "reference"' in capsys.readouterr().out
    assert main(["bench", "--gpus", "2"]) == 2


def test_trace_replay_options():
    """``bin/trace_run``: the four options of its contract, and the three beside them."""
    from sglang_rs_b200.engine.replay import DEFAULT_MAX_LIVE, PAGE_SIZE, build_parser as replay_parser
    args = replay_parser().parse_args(["--model", "/m", "--dtype", "float32", "--out", "/o", "--max-tokens", "640"])
    assert (args.model, args.dtype, args.out, args.max_tokens) == ("/m", "float32", "/o", 640)
    assert (args.page_size, args.max_live, args.radix) == (PAGE_SIZE, DEFAULT_MAX_LIVE, False) and DEFAULT_MAX_LIVE == 4
    args = replay_parser().parse_args(["--model", "/m", "--dtype", "bfloat16", "--out", "/o", "--max-tokens", "64",
                                       "--max-live", "150", "--radix", "--page-size", "8"])
    assert (args.max_live, args.radix, args.page_size) == (150, True, 8)
    with pytest.raises(SystemExit):
        replay_parser().parse_args(["--model", "/m", "--dtype", "float16", "--out", "/o", "--max-tokens", "64"])
