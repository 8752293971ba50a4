"""Replay of the same requests cut in different ways, in 32-bit and in bfloat16, against the
plain implementation: whole; most in one step and the last 32 one by one; in portions of
changing size; mixed with other requests on so few pages that they are used again."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model as pm
import replay_helpers as rh

pytestmark = pytest.mark.gpu

CASES = {
    # config, request lengths, page size
    "A": (pm.TINY_A, (5, 17, 33, 64, 200, 131), 16),
    "B": (pm.TINY_B, (7, 40, 90, 128, 65, 33), 8),
    "C": (pm.TINY_C, (3, 300, 47, 600, 258, 513), 16),
    # head_dim 128 / 64: in bfloat16 these run the tensor-core attention kernels and the tcgen05 product
    "D": (pm.TINY_D, (2, 129, 700, 64, 385, 257), 16),
    "E": (pm.TINY_E, (65, 130, 31, 400, 5, 90, 200, 33), 32),
    # head_dim 18: even, no multiple of 16 (scalar paths of the rope kernel, a ragged last lane of the attention)
    "F": (pm.TINY_F, (4, 150, 61, 300, 97), 4),
}
DTYPES = {"float32": (torch.float32, rh.FP32_TOLERANCE), "bfloat16": (torch.bfloat16, rh.BF16_TOLERANCE)}


@pytest.fixture(scope="module")
def prepared(tmp_path_factory):
    cache = {}

    def get(case, dtype_name):
        key = (case, dtype_name)
        if key not in cache:
            config, lengths, page = CASES[case]
            folder = rh.make_folder(tmp_path_factory.mktemp(f"{case}_{dtype_name}"), "model", config, seed=7,
                                    dtype=DTYPES[dtype_name][0])
            requests = rh.random_requests(config, lengths, seed=3)
            cache[key] = (folder, requests, rh.oracle(folder, requests), page)
        return cache[key]
    return get


def check(rows, expected, tolerance, requests, what):
    assert {rid: len(v) for rid, v in rows.items()} == {rid: len(t) for rid, t in requests.items()}
    bad = rh.first_bad(rows, expected, tolerance)
    worst, where = rh.worst_error(rows, expected)
    print(f"{what}: worst error {worst:.3e} of scale at {where}")
    assert bad is None, f"{what}: first wrong row: request {bad[0]} position {bad[1]} error {bad[2]:.3e} (tolerance {tolerance})"


@pytest.mark.parametrize("page", [1, 8, 64, 128, 256])
def test_other_page_sizes_of_the_tensor_core_kernels(prepared, page):
    """Head_dim 128 in bfloat16 with pages of 1 (the reference's default), 8 and 64 tokens (many pages,
    several, or one per 64-key block of the tcgen05 attention) and of 128 and 256 (which that kernel
    refuses: the mma.sync kernel takes the portions), portions mixed with decoded tokens."""
    folder, requests, expected, _ = prepared("D", "bfloat16")
    trace = rh.trace_mixed(requests, seed=4)
    rows, session = rh.run_in_process(folder, "bfloat16", trace, max_tokens=rh.max_tokens_of(trace, max(64, page)),
                                      page_size=page)           # pages larger than 64 round a request up to their own size
    check(rows, expected, rh.BF16_TOLERANCE, requests, f"D/bfloat16/mixed/page {page}")


@pytest.mark.parametrize("dtype_name", list(DTYPES))
@pytest.mark.parametrize("case", list(CASES))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cut_does_not_matter(prepared, case, dtype_name, mode):
    folder, requests, expected, page = prepared(case, dtype_name)
    trace = {"whole": rh.trace_whole, "tail": rh.trace_tail_by_one, "portions": rh.trace_portions,
             "mixed": lambda r: rh.trace_mixed(r, seed=11)}[mode](requests)
    rows, session = rh.run_in_process(folder, dtype_name, trace, page_size=page)
    check(rows, expected, DTYPES[dtype_name][1], requests, f"{case}/{dtype_name}/{mode}")
    if mode == "mixed":
        # pages that one request gave back were handed to another
        shared = [owners for owners in session.page_owners.values() if len(owners) > 1]
        assert len(shared) >= 3, "no page was used again; the trace does not test stale contents"


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_bfloat16_and_float32_cuts_agree_with_each_other(prepared, dtype_name):
    """Between two cuts of the same engine the difference is rounding only, far below the
    distance to the oracle in bfloat16."""
    folder, requests, expected, page = prepared("C", dtype_name)
    whole, _ = rh.run_in_process(folder, dtype_name, rh.trace_whole(requests), page_size=page)
    mixed, _ = rh.run_in_process(folder, dtype_name, rh.trace_mixed(requests, seed=5), page_size=page)
    as_expected = {rid: np.stack([whole[rid][p] for p in range(len(t))]).astype(np.float64) for rid, t in requests.items()}
    worst, where = rh.worst_error(mixed, as_expected)
    print(f"C/{dtype_name}: mixed against whole: {worst:.3e} at {where}")
    assert worst <= (2e-5 if dtype_name == "float32" else 2e-2)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
@pytest.mark.parametrize("case", ["A", "C"])
def test_captured_decode_steps_equal_eager_ones(prepared, case, dtype_name):
    """Decoded tokens replayed from CUDA graphs (padded to a bucket of rows) against the same
    steps launched one kernel at a time."""
    folder, requests, expected, page = prepared(case, dtype_name)
    for trace in (rh.trace_tail_by_one(requests), rh.trace_mixed(requests, seed=21)):
        eager, _ = rh.run_in_process(folder, dtype_name, trace, page_size=page, graphs=False)
        captured, session = rh.run_in_process(folder, dtype_name, trace, page_size=page, graphs=True)
        assert session.runner.graphs is not None and session.runner.graphs.replays > 30
        as_expected = {rid: np.stack([eager[rid][p] for p in range(len(t))]).astype(np.float64)
                       for rid, t in requests.items()}
        worst, where = rh.worst_error(captured, as_expected)
        print(f"{case}/{dtype_name}: captured against eager: {worst:.3e} at {where}")
        assert worst <= (0.0 if dtype_name == "float32" else 1e-2)
        check(captured, expected, DTYPES[dtype_name][1], requests, f"{case}/{dtype_name}/captured")


@pytest.mark.parametrize("dtype_name", list(DTYPES))
def test_replay_with_the_prefix_tree(tmp_path, dtype_name):
    """Tiny B, pages of 8: a second prompt shares 24 tokens with the first and is fed whole; it starts at
    position 24 on the first one's three pages, and its rows from 24 on equal the oracle's rows of the whole
    prompt.  A prompt that is known entirely still computes what lies behind its last whole page but one token
    (40 known tokens: 4 pages taken).  A third kind arrives in two portions: only the first is matched."""
    stored, tolerance = DTYPES[dtype_name]
    folder = rh.make_folder(tmp_path, "radix", pm.TINY_B, seed=41, dtype=stored)
    base = list(rh.random_requests(pm.TINY_B, (40,), seed=12).values())[0]
    requests = {"a": base,
                "b": base[:24] + list(rh.random_requests(pm.TINY_B, (16,), seed=13).values())[0],
                "c": list(base),
                "d": base[:24] + list(rh.random_requests(pm.TINY_B, (30,), seed=14).values())[0]}
    expected = rh.oracle(folder, requests)
    whole = lambda rid: {"id": rid, "tokens": requests[rid], "want": list(range(len(requests[rid])))}  # noqa: E731
    trace = [{"step": 0, "entries": [whole("a")], "end": []},
             {"step": 1, "entries": [whole("b")], "end": []},
             {"step": 2, "entries": [whole("c"), {"id": "d", "tokens": requests["d"][:30], "want": list(range(30))}],
              "end": ["a"]},
             {"step": 3, "entries": [{"id": "d", "tokens": requests["d"][30:], "want": list(range(24))}],
              "end": ["b", "c", "d"]}]
    from sglang_rs_b200.engine.replay import ReplaySession
    session = ReplaySession(folder, dtype_name, 512, page_size=8, radix=True)
    outputs, tables = [], {}
    for step in trace:
        outputs.append(session.run(step))
        for rid, handle in session.handles.items():
            tables[rid] = handle.table(("kv", None))
        session.cache.check_invariants()
    assert session.cached_tokens == {"a": 0, "b": 24, "c": 32, "d": 24}
    assert tables["b"][:3] == tables["a"][:3] and tables["b"][3] != tables["a"][3]     # the same physical pages
    assert tables["c"][:4] == tables["a"][:4] and tables["d"][:3] == tables["a"][:3]
    rows = rh.collect(trace, outputs)
    computed = {}
    for rid, by_pos in rows.items():
        skipped = session.cached_tokens[rid]
        assert all(np.isnan(by_pos[p]).all() for p in range(skipped)), "rows inside the cached prefix are not computed"
        computed[rid] = {p: row for p, row in by_pos.items() if p >= skipped}
        assert len(computed[rid]) == len(requests[rid]) - skipped
    bad = rh.first_bad(computed, expected, tolerance)
    worst, where = rh.worst_error(computed, expected)
    print(f"B/{dtype_name}/prefix tree: worst error {worst:.3e} at {where}")
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} error {bad[2]:.3e}"
    tree = session.cache.prefix_tree
    assert tree.hits == 3 and not session.handles
    allocator = session.cache.allocators[("kv", None)]
    assert allocator.free_count + tree.pages_held == allocator.num_pages
    # without the tree the same trace computes every row, and the rows behind the prefix agree with those above
    plain_rows, _ = rh.run_in_process(folder, dtype_name, trace, max_tokens=512, page_size=8)
    for rid in computed:
        for p, row in computed[rid].items():
            err = float(np.abs(row.astype(np.float64) - plain_rows[rid][p]).max()) / float(np.abs(expected[rid]).max())
            assert err <= (2e-5 if dtype_name == "float32" else 2e-2), (rid, p, err)


@pytest.mark.parametrize("dtype_name", list(DTYPES))
@pytest.mark.parametrize("case", ["A", "C", "D", "F"])
def test_a_step_in_one_native_call_equals_the_step_part_by_part(prepared, case, dtype_name):
    """The step executor launches what the parts would launch one by one: the same kernels with the same
    arguments, so the logits are equal bit for bit, in both dtypes, captured or not, on a trace that mixes
    portions with decoded tokens (C has biases and one kv head, D the tensor-core kernels, F head_dim 18)."""
    folder, requests, expected, page = prepared(case, dtype_name)
    for trace, graphs in ((rh.trace_mixed(requests, seed=31), False), (rh.trace_tail_by_one(requests), True)):
        native, session = rh.run_in_process(folder, dtype_name, trace, page_size=page, graphs=graphs, native_step=True)
        assert session.model.native is not None
        by_parts, other = rh.run_in_process(folder, dtype_name, trace, page_size=page, graphs=graphs, native_step=False)
        assert other.model.native is None
        for rid in by_parts:
            for p, row in by_parts[rid].items():
                assert np.array_equal(row, native[rid][p]), (case, dtype_name, graphs, rid, p)
        check(native, expected, DTYPES[dtype_name][1], requests, f"{case}/{dtype_name}/native step")


def test_trace_run_program(prepared, tmp_path):
    """The program itself, as a user calls it: steps on standard input, files out."""
    folder, requests, expected, page = prepared("A", "float32")
    trace = rh.trace_mixed(requests, seed=2)
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    process = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
         "--out", str(out), "--max-tokens", str(rh.max_tokens_of(trace))],
        input="\n".join(json.dumps(s) for s in trace) + "\n", capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    assert process.stdout.split() == [x for s in trace for x in ("done", str(s["step"]))]
    vocab = pm.TINY_A["vocab_size"]
    outputs = []
    for s in trace:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4")
            assert data.size == wanted * vocab
            outputs.append(data.reshape(wanted, vocab))
        else:
            assert not path.exists()
            outputs.append(None)
    check(rh.collect(trace, outputs), expected, rh.FP32_TOLERANCE, requests, "trace_run A/float32/mixed")


@pytest.mark.parametrize("dtype_name", ["bfloat16", "float32"])
def test_layer_sizes_of_the_8b_shape(tmp_path, dtype_name):
    """Layers with the benchmark's layer sizes (hidden 4096, 32/8 heads of 128, inner 12288; two of them in
    32-bit, one in bfloat16) and a vocabulary of 32,000: the products are cut along K as in the benchmark and the
    attention kernels see 4 query heads per kv head.  Prompt in one step, then tokens one by one across a key split."""
    config = dict(pm.TINY_D, num_hidden_layers=2 if dtype_name == "float32" else 1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                  head_dim=128, intermediate_size=12288, vocab_size=32000, max_position_embeddings=512)
    stored = DTYPES[dtype_name][0]
    folder = rh.make_folder(tmp_path, "big", config, seed=5, dtype=stored)
    requests = rh.random_requests(config, (150, 40), seed=9)
    cfg, weights = pm.load_folder(folder)
    # 32-bit is held to the bound of the tiny models, against a 64-bit oracle; for bfloat16 a 32-bit oracle does
    oracle_dtype = torch.float64 if dtype_name == "float32" else torch.float32
    expected = {rid: pm.plain_forward(cfg, weights, toks, dtype=oracle_dtype).double().numpy()
                for rid, toks in requests.items()}
    trace = rh.trace_tail_by_one(requests, tail=30) if dtype_name == "bfloat16" else rh.trace_portions(requests)
    rows, _ = rh.run_in_process(folder, dtype_name, trace)
    tolerance = DTYPES[dtype_name][1]
    check(rows, expected, tolerance, requests, f"8B layer sizes/{dtype_name}")
