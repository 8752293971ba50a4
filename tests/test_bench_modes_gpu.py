"""The side modes of bench.py on a small case: they are what the figures under profiles/ come from, so they have to
keep running."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*arguments):
    process = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *arguments], capture_output=True, text=True,
                             timeout=900, cwd=ROOT)
    assert process.returncode == 0, (process.stdout + process.stderr)[-3000:]
    return json.loads(process.stdout.strip().splitlines()[-1]), process.stderr


def test_the_timeline_of_a_decode_step_names_every_kernel_of_a_layer():
    line, table = run_bench("--mode", "timeline", "--shape", "qwen3-1.7b", "--layers", "2", "--batch", "2", "--context", "256")
    assert line["mode"] == "timeline" and line["records"] > 0
    for kernel in ("add + norm", "product", "rope + page write", "decode attention"):
        for what in ("first block starts", "wait for the kernels ahead returns", "block leaves"):
            assert f"{kernel}: {what}" in table, (kernel, what)
    # a kernel's wait cannot return before its first block has started, nor a block leave before that
    firsts = {}
    for row in table.splitlines():
        parts = row.split(None, 3)
        if len(parts) == 4 and ":" in parts[3] and parts[0].replace(".", "").isdigit():
            firsts.setdefault(parts[3].strip(), float(parts[0]))
    assert firsts["add + norm: first block starts"] <= firsts["add + norm: wait for the kernels ahead returns"] \
        <= firsts["add + norm: block leaves"]


def test_the_timeline_of_a_prefill_step_lists_the_attention_tile_by_tile():
    line, table = run_bench("--mode", "timeline", "--only-prefill", "--prefill-tokens", "512", "--shape", "qwen3-1.7b",
                            "--layers", "2")
    assert line["mode"] == "timeline" and line["attention_us_last_layer"] > 0
    assert "blocks on" in table and table.count("\n") >= 5          # a header, four tiles of 128 rows, the summary


def test_kernel_classes_ablation_serving_and_the_comparison_with_cublas_on_a_small_case():
    line, _ = run_bench("--mode", "kernels", "--shape", "qwen3-1.7b", "--layers", "2", "--prefill-tokens", "256", "--batch", "2",
                        "--context", "128")
    assert line["mode"] == "kernels" and line["prefill"]["gemm"] > 0 and line["decode"]["attention_decode"] > 0
    line, _ = run_bench("--mode", "ablate", "--shape", "qwen3-1.7b", "--layers", "2", "--batch", "2", "--context", "128", "--steps", "4")
    assert line["mode"] == "ablate" and set(line["us_saved_per_layer_by_leaving_out"]) >= {"norm", "rope", "attention", "qkv"}
    line, _ = run_bench("--mode", "serve", "--shape", "qwen3-1.7b", "--layers", "2", "--requests", "6")
    assert line["mode"] == "serve" and line["requests"] == 6 and line["value"] > 0 and line["preemptions"] >= 0
    line, _ = run_bench("--mode", "compare-cublas", "--shape", "qwen3-1.7b", "--rows", "8,128")
    assert line["mode"] == "compare-cublas"
    by_key = {(entry["product"], entry["rows"]): entry for entry in line["products"]}
    assert by_key[("qkv", 8)]["own_us"] > 0 and by_key[("down", 128)]["cublas_us"] > 0
