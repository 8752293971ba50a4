"""Generation through the entry point, long decoding, the first tokens of a sequence, each
part alone, and an architecture defined here (a mixer with state of its own, layers of
different kinds, a layer called twice, a layer that reads another layer's cache) that is
registered, built and stepped without a change to the framework's files."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_model as pm
import replay_helpers as rh

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_greedy_margin(config, weights, prompt, got, limit):
    """Every generated token is the plain argmax, or (bfloat16) within ``limit`` of it."""
    tokens = list(prompt)
    for token in got:
        logits = pm.plain_forward(config, weights, tokens)[-1]
        best = int(torch.argmax(logits))
        assert float(logits[best] - logits[token]) <= limit * float(logits.abs().max()), (prompt[:4], got, token, best)
        tokens.append(token)


# ------------------------------------------------------------------------------ generation
@pytest.mark.parametrize("dtype_name,stored,limit", [("float32", torch.float32, 0.0), ("bfloat16", torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("config,page,chunk,pool", [(pm.TINY_A, 16, 16, 512), (pm.TINY_B, 8, 16, 160), (pm.TINY_C, 16, 50, 400)])
def test_greedy_generation_through_the_entry_point(tmp_path, config, page, chunk, pool, dtype_name, stored, limit):
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", config, seed=21, dtype=stored)
    cfg, weights = pm.load_folder(folder)
    lengths = (5, 17, 33, 64) if config is not pm.TINY_B else (7, 40, 90)
    prompts = list(rh.random_requests(config, lengths, seed=8).values())
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=page, max_total_tokens=pool,
                    max_running_requests=3, chunked_prefill_size=chunk)
    results = engine.generate(prompts, {"max_new_tokens": 16})
    for prompt, result in zip(prompts, results):
        assert result["finished"] and result["finish_reason"] == "length" and len(result["output_ids"]) == 16
        plain_greedy_margin(cfg, weights, prompt, result["output_ids"], limit)
    if dtype_name == "float32":
        assert [r["output_ids"] for r in results] == [pm.plain_greedy(cfg, weights, p, 16) for p in prompts]
    # the same prompts one at a time, with another budget: the same tokens
    again = Engine(model_path=folder, dtype=dtype_name, page_size=page, max_total_tokens=pool,
                   max_running_requests=1, chunked_prefill_size=7)
    if dtype_name == "float32":
        assert [again.generate(p, {"max_new_tokens": 16})["output_ids"] for p in prompts] == [r["output_ids"] for r in results]
    engine.cache.check_invariants()
    assert engine.flush_cache()                          # cached prompt pages are the only ones still held
    assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())


def test_logits_of_a_trace_through_the_engine(tmp_path):
    """`Engine.forward_logits` takes the step records of trace replay: the engine's own model, cache and
    step function, beside its scheduler."""
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_A, seed=4, dtype=torch.float32)
    cfg, weights = pm.load_folder(folder)
    engine = Engine(model_path=folder, dtype="float32", max_total_tokens=256)
    tokens = rh.random_requests(pm.TINY_A, (40,), seed=1)["r0"]
    want = pm.plain_forward(cfg, weights, tokens).numpy()
    first = engine.forward_logits({"entries": [{"id": "t", "tokens": tokens[:33], "want": [0, 32]}], "end": []})
    assert engine.forward_logits({"entries": [{"id": "t", "tokens": tokens[33:39], "want": []}]}) is None
    last = engine.forward_logits({"entries": [{"id": "t", "tokens": tokens[39:], "want": [0]}], "end": ["t"]})
    scale = abs(want).max()
    for got, position in ((first[0], 0), (first[1], 32), (last[0], 39)):
        assert abs(got - want[position]).max() / scale < rh.FP32_TOLERANCE
    assert engine.generate(tokens[:5], {"max_new_tokens": 4})["output_ids"] == pm.plain_greedy(cfg, weights, tokens[:5], 4)
    engine.cache.check_invariants()


def test_preemption_on_a_small_pool_gives_the_same_tokens(tmp_path):
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_A, seed=4, dtype=torch.float32)
    cfg, weights = pm.load_folder(folder)
    prompts = list(rh.random_requests(pm.TINY_A, (40, 35, 50), seed=2).values())
    engine = Engine(model_path=folder, dtype="float32", page_size=16, max_total_tokens=160, max_running_requests=3,
                    chunked_prefill_size=64)
    results = engine.generate(prompts, {"max_new_tokens": 40})
    assert engine.scheduler.stats["preemptions"] >= 1
    assert [r["output_ids"] for r in results] == [pm.plain_greedy(cfg, weights, p, 40) for p in prompts]


@pytest.mark.parametrize("overlap", [True, False])
def test_many_preemptions_with_long_prompts_change_no_token(overlap):
    """Sixteen requests with prompts of up to 1,500 tokens on a pool that holds a fifth of them (layers of 1,024 wide,
    heads of 128: portions of 512 rows go through the kernels for many rows): the requests are preempted dozens of
    times, their prompts computed again in other portions and beside other rows, and in 32-bit every token must be
    the one that a pool without pressure gives."""
    import random
    from sglang_rs_b200 import Engine
    config = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 1024,
              "num_attention_heads": 8, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 1536,
              "vocab_size": 3001, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
              "max_position_embeddings": 4096, "hidden_act": "silu", "attention_bias": False}
    rng = random.Random(5)
    prompts = [[rng.randrange(config["vocab_size"]) for _ in range(rng.choice([17, 130, 300, 700, 1500]))] for _ in range(16)]
    new_tokens = [rng.choice([8, 40, 90]) for _ in prompts]

    def run(pool):
        engine = Engine(config=config, random_weights=True, seed=1, dtype="float32", page_size=16, max_total_tokens=pool,
                        max_running_requests=12, chunked_prefill_size=512, disable_overlap_schedule=not overlap)
        ids = [engine.add_request(p, {"max_new_tokens": n, "ignore_eos": True}) for p, n in zip(prompts, new_tokens)]
        tokens = {i: [] for i in ids}
        while engine.scheduler.has_work or engine._in_flight is not None:
            for output in engine.step(overlap=overlap):
                tokens[output.request_id].extend(output.token_ids)
        for output in engine.drain():
            tokens[output.request_id].extend(output.token_ids)
        engine.cache.check_invariants()
        return [tokens[i] for i in ids], engine.scheduler.stats["preemptions"]

    at_ease, none = run(40000)
    pressed, preemptions = run(2400)
    assert none == 0 and preemptions >= 10
    assert [len(t) for t in pressed] == new_tokens
    assert pressed == at_ease


@pytest.mark.parametrize("dtype_name,stored,limit", [("float32", torch.float32, 0.0), ("bfloat16", torch.bfloat16, 3e-2)])
def test_shared_prefix_is_reused_and_changes_nothing(tmp_path, dtype_name, stored, limit):
    """Two prompts share 24 tokens (3 pages of 8); the second starts from the first one's pages.
    A prompt that is cached entirely still computes its last page's tokens."""
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_B, seed=31, dtype=stored)
    cfg, weights = pm.load_folder(folder)
    base = list(rh.random_requests(pm.TINY_B, (90,), seed=12).values())[0]
    other = base[:24] + list(rh.random_requests(pm.TINY_B, (16,), seed=13).values())[0]
    engine = Engine(model_path=folder, dtype=dtype_name, page_size=8, max_total_tokens=400, chunked_prefill_size=16)
    first = engine.generate(base[:40], {"max_new_tokens": 6})
    assert first["cached_tokens"] == 0
    second = engine.generate(other, {"max_new_tokens": 6})
    assert second["cached_tokens"] == 24
    third = engine.generate(base[:40], {"max_new_tokens": 6})
    assert third["cached_tokens"] == 32                   # 40 tokens known; (40 - 1) // 8 pages are taken
    for prompt, result in ((base[:40], first), (other, second), (base[:40], third)):
        plain_greedy_margin(cfg, weights, prompt, result["output_ids"], limit)
    assert third["output_ids"] == first["output_ids"]
    fresh = Engine(model_path=folder, dtype=dtype_name, page_size=8, max_total_tokens=400, chunked_prefill_size=16,
                   disable_radix_cache=True)
    assert fresh.cache.prefix_tree is None
    if dtype_name == "float32":
        assert fresh.generate(other, {"max_new_tokens": 6})["output_ids"] == second["output_ids"]
    # cached pages make room when the pool is needed: a long request evicts them
    long = list(rh.random_requests(pm.TINY_B, (100,), seed=14).values())
    many = engine.generate(long * 3, {"max_new_tokens": 20})
    assert all(r["finished"] for r in many)
    engine.cache.check_invariants()


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(tmp_path):
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_B, seed=6, dtype=torch.float32)
    prompts = list(rh.random_requests(pm.TINY_B, (7, 40, 24), seed=5).values())
    params = [{"max_new_tokens": 20, "temperature": 0.7, "seed": 100 + i} for i in range(3)]
    engine = Engine(model_path=folder, dtype="float32", page_size=8, max_total_tokens=400, chunked_prefill_size=16)
    together = [r["output_ids"] for r in engine.generate(prompts, params)]
    alone = [engine.generate(p, q)["output_ids"] for p, q in zip(prompts, params)]
    assert together == alone
    other = engine.generate(prompts[0], dict(params[0], seed=999))["output_ids"]
    assert other != together[0]
    # every sampled token is what the plain sampler picks from the plain logits with the same uniform number
    from sglang_rs_b200.sampling import RequestRandom
    cfg, weights = pm.load_folder(folder)
    rng = RequestRandom("x", 100)
    tokens = list(prompts[0])
    for token in together[0]:
        logits = pm.plain_forward(cfg, weights, tokens)[-1]
        u = rng.next_unit()
        want = pm.plain_temperature_sample(logits, 0.7, float(np.float32(u)))
        if token != want:       # only a tie of the running sum at rounding may move the pick by one place
            p = torch.softmax(logits / 0.7, 0)
            assert abs(token - want) == 1 and abs(float(torch.cumsum(p, 0)[min(token, want)]) - u) < 1e-4
        tokens.append(token)


@pytest.mark.parametrize("use_graphs", [True, False])
def test_overlapped_steps_give_the_same_tokens(tmp_path, use_graphs):
    """With ``overlap`` a step is launched before the tokens of the step before are read: decoded
    tokens travel on the device, finished requests get one row in vain.  Requests that stop at
    different times (stop tokens, lengths), requests that join later, temperature sampling, a
    request whose sampling needs the host, and a pool so small that requests are preempted: the
    tokens are those of the plain loop."""
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_B, seed=14, dtype=torch.float32)
    cfg, weights = pm.load_folder(folder)
    prompts = list(rh.random_requests(pm.TINY_B, (9, 30, 17, 41, 5, 26), seed=3).values())
    greedy = [pm.plain_greedy(cfg, weights, p, 24) for p in prompts]
    params = [{"max_new_tokens": 24},
              {"max_new_tokens": 24, "stop_token_ids": [greedy[1][6]]},
              {"max_new_tokens": 11},
              {"max_new_tokens": 20, "temperature": 0.8, "seed": 4},
              {"max_new_tokens": 1},
              {"max_new_tokens": 24, "stop_token_ids": [greedy[5][15]]}]

    def run(overlap, pool, late=(), extra=None):
        engine = Engine(model_path=folder, dtype="float32", page_size=8, max_total_tokens=pool, max_running_requests=4,
                        chunked_prefill_size=24, disable_cuda_graph=not use_graphs)
        chosen = dict(enumerate(params))
        if extra:
            chosen.update(extra)
        ids = {}
        for i, prompt in enumerate(prompts):
            if i not in late:
                ids[i] = engine.add_request(prompt, chosen[i])
        got = {i: [] for i in range(len(prompts))}
        by_id = lambda rid: next(i for i, v in ids.items() if v == rid)
        steps = 0
        while engine.scheduler.has_work or engine._in_flight is not None or len(ids) < len(prompts):
            if steps == 5:
                for i in late:
                    ids[i] = engine.add_request(prompts[i], chosen[i])
            for output in engine.step(overlap=overlap):
                got[by_id(output.request_id)] += output.token_ids
            steps += 1
            assert steps < 500
        engine.cache.check_invariants()
        assert engine.flush_cache()
        assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())
        return [got[i] for i in range(len(prompts))], engine.scheduler.stats["preemptions"]

    plain, _ = run(False, 600)
    assert plain[0] == greedy[0] and plain[2] == greedy[2][:11] and plain[4] == greedy[4][:1]
    assert plain[1] == greedy[1][:greedy[1].index(greedy[1][6]) + 1]
    assert run(True, 600) == (plain, 0)
    assert run(True, 600, late=(2, 5))[0] == plain
    # a request with top-k among them: its steps wait for the host, the tokens stay the same
    top = {0: {"max_new_tokens": 24, "temperature": 1.0, "top_k": 1}}
    assert run(True, 600, extra=top)[0] == plain
    # so few pages that requests are preempted and recomputed
    tight, preemptions = run(True, 104)
    assert tight == plain and preemptions > 0


def test_stop_tokens_top_k_and_penalties(tmp_path):
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_A, seed=9, dtype=torch.float32)
    cfg, weights = pm.load_folder(folder)
    prompt = list(rh.random_requests(pm.TINY_A, (12,), seed=1).values())[0]
    greedy = pm.plain_greedy(cfg, weights, prompt, 8)
    engine = Engine(model_path=folder, dtype="float32", max_total_tokens=256)
    stopped = engine.generate(prompt, {"max_new_tokens": 8, "stop_token_ids": [greedy[3]]})
    first = greedy.index(greedy[3])
    assert stopped["output_ids"] == greedy[:first + 1] and stopped["finish_reason"] == "stop"
    ignored = engine.generate(prompt, {"max_new_tokens": 8, "stop_token_ids": [greedy[3]], "ignore_eos": True})
    assert ignored["output_ids"] == greedy
    assert engine.generate(prompt, {"max_new_tokens": 8, "temperature": 1.0, "top_k": 1})["output_ids"] == greedy
    # top-k 3: every token is among the three best of the plain logits
    out = engine.generate(prompt, {"max_new_tokens": 12, "temperature": 1.5, "top_k": 3, "seed": 5})["output_ids"]
    tokens = list(prompt)
    for token in out:
        logits = pm.plain_forward(cfg, weights, tokens)[-1]
        assert token in torch.topk(logits, 3).indices.tolist()
        tokens.append(token)
    # a strong repetition penalty: the penalised greedy path of the plain implementation
    out = engine.generate(prompt, {"max_new_tokens": 10, "repetition_penalty": 1.8, "presence_penalty": 0.5,
                                   "frequency_penalty": 0.3})["output_ids"]
    tokens = list(prompt)
    for token in out:
        logits = pm.plain_apply_penalties(pm.plain_forward(cfg, weights, tokens)[-1], tokens, 0.3, 0.5, 1.8)
        assert token == int(torch.argmax(logits))
        tokens.append(token)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.generate([1, 2, 99999], {"max_new_tokens": 2})


def test_command_line(tmp_path):
    folder = rh.make_folder(tmp_path, "m", pm.TINY_A, seed=3, dtype=torch.float32)
    cfg, weights = pm.load_folder(folder)
    process = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "sglang-rs"), "generate", f"--model-path={folder}", "--device", "cuda",
         "--dtype", "float32", "--input-ids", "5,17,3", "--input-ids", "9 8 7 6", "--max-new-tokens", "5",
         "--max-total-tokens", "256", "--some-unknown-flag"],
        capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    lines = [json.loads(line) for line in process.stdout.strip().splitlines()]
    assert [l["input_ids"] for l in lines] == [[5, 17, 3], [9, 8, 7, 6]]
    assert [l["output_ids"] for l in lines] == [pm.plain_greedy(cfg, weights, p, 5) for p in ([5, 17, 3], [9, 8, 7, 6])]
    refused = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "sglang-rs"), "generate", "--model-path", folder,
                              "--device", "cpu", "--input-ids", "1"], capture_output=True, text=True, timeout=600)
    assert refused.returncode != 0 and "CUDA only" in refused.stderr


# ------------------------------------------------------------------------------ long decoding, first tokens
@pytest.mark.parametrize("dtype_name,stored,tolerance", [("float32", torch.float32, rh.FP32_TOLERANCE),
                                                         ("bfloat16", torch.bfloat16, rh.BF16_TOLERANCE)])
def test_long_decoding_and_first_tokens(tmp_path, dtype_name, stored, tolerance):
    """A prompt of two tokens, then 600 tokens decoded one by one (three key splits, many
    pages); beside it a request whose every position from the very first is checked."""
    folder = rh.make_folder(tmp_path, "m", pm.TINY_C, seed=13, dtype=stored)
    requests = rh.random_requests(pm.TINY_C, (602, 9), seed=17)
    expected = rh.oracle(folder, requests)
    long, short = requests["r0"], requests["r1"]
    trace = [{"entries": [{"id": "r0", "tokens": long[:2], "want": [0, 1]}], "end": []}]
    for p in range(2, len(long)):
        entries = [{"id": "r0", "tokens": [long[p]], "want": [0]}]
        if p - 2 < len(short):
            entries.append({"id": "r1", "tokens": [short[p - 2]], "want": [0]})     # token by token from position 0
        trace.append({"entries": entries, "end": ["r1"] if p - 2 == len(short) - 1 else []})
    trace[-1]["end"] = ["r0"]
    for i, step in enumerate(trace):
        step["step"] = i
    rows, _ = rh.run_in_process(folder, dtype_name, trace)
    bad = rh.first_bad(rows, expected, tolerance)
    print("long decoding:", rh.worst_error(rows, expected))
    assert bad is None, bad
    assert len(rows["r0"]) == 602 and len(rows["r1"]) == 9


# ------------------------------------------------------------------------------ parts alone
def part_context(needs, entries_tokens, dtype, page_size=8, scratch=()):
    """A cache manager and a flattened step for single parts: ``entries_tokens`` is a list of
    (request id, start length, token count)."""
    from sglang_rs_b200.cache import CacheManager
    from sglang_rs_b200.engine import StepEntry, StepPlanner
    cache = CacheManager(needs, page_size=page_size, max_tokens=1024, max_requests=8, device=DEV, dtype=dtype)
    planner = StepPlanner(cache, DEV, dtype, scratch)
    return cache, planner


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    from sglang_rs_b200.engine import StepEntry
    from sglang_rs_b200.parts import (AttentionNames, GatedMlp, GatedMlpNames, GroupedQueryAttention, OutputHead,
                                      PreNormBlock, RmsNorm, RotaryEncoding, TokenEmbedding)
    g = torch.Generator().manual_seed(0)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    hidden, inner, n_q, n_kv, d, vocab, eps, theta = 40, 56, 6, 2, 16, 77, 1e-5, 777.0

    def seen(t):
        return t.to(dtype).double()

    def close(got, want, what):
        err = float((got.double().cpu() - want).abs().max() / want.abs().max())
        assert err <= tol, f"{what}: {err:.3e}"

    w = {"n1": 1 + 0.1 * torch.randn(hidden, generator=g), "n2": 1 + 0.1 * torch.randn(hidden, generator=g),
         "q": torch.randn(n_q * d, hidden, generator=g) * 0.2, "k": torch.randn(n_kv * d, hidden, generator=g) * 0.2,
         "v": torch.randn(n_kv * d, hidden, generator=g) * 0.2, "o": torch.randn(hidden, n_q * d, generator=g) * 0.2,
         "qn": 1 + 0.1 * torch.randn(d, generator=g), "kn": 1 + 0.1 * torch.randn(d, generator=g),
         "gate": torch.randn(inner, hidden, generator=g) * 0.2, "up": torch.randn(inner, hidden, generator=g) * 0.2,
         "down": torch.randn(hidden, inner, generator=g) * 0.2, "emb": torch.randn(vocab, hidden, generator=g),
         "head": torch.randn(vocab, hidden, generator=g) * 0.2}
    norm1, norm2 = RmsNorm(hidden, eps, "n1"), RmsNorm(hidden, eps, "n2")
    rope = RotaryEncoding(d, theta)
    attention = GroupedQueryAttention(hidden, n_q, n_kv, d, 1 / math.sqrt(d), rope,
                                      AttentionNames("q", "k", "v", "o", "qn", "kn"), qk_norm_eps=eps)
    mlp = GatedMlp(hidden, inner, "silu", GatedMlpNames("gate", "up", "down"))
    block = PreNormBlock(norm1, attention, norm2, mlp)
    embedding = TokenEmbedding(vocab, hidden, "emb")
    head, tied = OutputHead(vocab, hidden, "head"), OutputHead(vocab, hidden, None, embedding)
    assert set(block.tensor_specs()) == {"n1", "n2", "q", "k", "v", "o", "qn", "kn", "gate", "up", "down"}
    for part in (block, embedding, head, tied):
        part.load(w, DEV, dtype)

    # rotary table: theta^(-2i/d) in 64-bit
    assert torch.equal(rope.fused_rotary().inv_freq.cpu(), pm.plain_inverse_frequencies(theta, d))

    # norm alone, with the pending sum
    residual, delta = torch.randn(5, hidden, generator=g), torch.randn(5, hidden, generator=g)
    res_d = residual.to(DEV)
    out = norm1.add_norm(res_d, delta.to(DEV, dtype), dtype)
    close(out, pm.plain_rms_norm(residual.double() + seen(delta), w["n1"].double(), eps), "norm")

    # feed-forward alone
    x = torch.randn(7, hidden, generator=g)
    mw = {k: seen(v) for k, v in w.items()}
    want = pm.plain_linear(pm.plain_silu_mul(pm.plain_linear(seen(x), mw["gate"]), pm.plain_linear(seen(x), mw["up"])), mw["down"])
    close(mlp.forward(None, x.to(DEV, dtype)), want, "mlp")

    # embedding and heads alone
    cache, planner = part_context([attention.cache_need()], None, dtype, scratch=[attention.split_scratch()])
    handle = cache.open("a")
    tokens = [3, 76, 0, 3, 19, 54, 8, 8, 41, 2, 33]
    cache.reserve(handle, len(tokens))
    ctx, _ = planner.flatten([StepEntry(handle, tokens, [])])
    emb = embedding.forward(ctx, ctx.token_ids)
    assert torch.equal(emb.cpu().double(), mw["emb"][tokens])
    close(head.forward(ctx, x.to(DEV, dtype)), pm.plain_linear(seen(x), mw["head"]), "head")
    close(tied.forward(ctx, x.to(DEV, dtype)), pm.plain_linear(seen(x), mw["emb"]), "tied head")
    assert head.forward(ctx, x.to(DEV, dtype)).dtype == torch.float32

    # attention alone: 11 tokens in one step, then 2 and 1 more, against the whole sequence
    def plain_attn(xs):
        pos = torch.arange(len(xs))
        q = pm.plain_rms_norm(pm.plain_linear(xs, mw["q"]).view(-1, n_q, d), w["qn"].double(), eps)
        k = pm.plain_rms_norm(pm.plain_linear(xs, mw["k"]).view(-1, n_kv, d), w["kn"].double(), eps)
        v = pm.plain_linear(xs, mw["v"]).view(-1, n_kv, d)
        inv = pm.plain_inverse_frequencies(theta, d)
        a = pm.plain_attention(pm.plain_rope_neox(q, pos, inv), pm.plain_rope_neox(k, pos, inv), v, 1 / math.sqrt(d))
        return pm.plain_linear(a.reshape(len(xs), -1), mw["o"])

    xs = torch.randn(14, hidden, generator=g)
    want = plain_attn(seen(xs))
    layer_cache = cache.layer_cache(0)
    got = [attention.forward(ctx, layer_cache, xs[:11].to(DEV, dtype))]
    cache.commit(handle, 11)
    for begin, end in ((11, 13), (13, 14)):
        cache.reserve(handle, end - begin)
        ctx, _ = planner.flatten([StepEntry(handle, [1] * (end - begin), [])])
        got.append(attention.forward(ctx, layer_cache, xs[begin:end].to(DEV, dtype)))
        cache.commit(handle, end - begin)
    close(torch.cat(got), want, "attention")

    # the block alone: (residual, delta) in, (residual, delta) out
    other = cache.open("b")
    cache.reserve(other, 6)
    ctx, _ = planner.flatten([StepEntry(other, [1] * 6, [])])
    h = torch.randn(6, hidden, generator=g)
    res, dlt = block.forward(ctx, layer_cache, h.to(DEV).clone(), None)
    a = plain_attn(pm.plain_rms_norm(h.double(), w["n1"].double(), eps).to(dtype).double())
    mid = h.double() + a
    normed = pm.plain_rms_norm(mid, w["n2"].double(), eps)
    ff = pm.plain_linear(pm.plain_silu_mul(pm.plain_linear(normed, mw["gate"]), pm.plain_linear(normed, mw["up"])), mw["down"])
    if dlt is None:                          # the last product's kernel added it to the residual stream
        total = res.double()
    else:
        total = res.double() + (dlt.double() if dlt.dim() == 2 else dlt.double().sum(0))
    close(total, mid + ff, "block")
    planner_error = planner.error_word
    from sglang_rs_b200 import ops
    ops.raise_on_error_word(planner_error)


# ------------------------------------------------------------------------------ an architecture defined here
TOY = {"architectures": ["ToyHybridForTests"], "hidden": 48, "vocab": 90, "heads": 4, "kv_heads": 2, "head_dim": 16,
       "inner": 64, "eps": 1e-5, "theta": 3000.0, "window": 11, "decay": 0.8, "max_positions": 400}


def register_toy(stateless=False):
    """Everything the toy needs is defined here; the framework's files are not touched."""
    from sglang_rs_b200 import ops
    from sglang_rs_b200.config import register_architecture
    from sglang_rs_b200.models import DecoderModel, LayerCall
    from sglang_rs_b200.parts import (AttentionNames, GatedMlp, GatedMlpNames, GroupedQueryAttention, Mixer,
                                      NoPositionEncoding, OutputHead, PreNormBlock, RequestState, RmsNorm,
                                      RotaryEncoding, TensorSpec, TokenEmbedding, matrix_to)

    class DecayingSumMixer(Mixer):
        """s_t = decay * s_{t-1} + W x_t; y_t = s_t.  The state s lives in the request's slot."""

        def __init__(self, hidden, decay, weight_name, on_device=False):
            self.hidden, self.decay, self.weight_name = hidden, decay, weight_name
            # with its decode step on the device (below) the mixer may be captured into a CUDA graph
            self.graph_safe = on_device

        def cache_need(self):
            return RequestState((self.hidden,), torch.float32)

        def tensor_specs(self):
            return {self.weight_name: TensorSpec((self.hidden, self.hidden))}

        def load(self, tensors, device, dtype):
            self.w = matrix_to(tensors[self.weight_name], device, dtype)

        def forward(self, ctx, cache, x):
            v = ops.linear(x, self.w).float()
            if self.graph_safe and all(b - a == 1 for a, b in zip(ctx.host_cu_rows, ctx.host_cu_rows[1:])):
                # one row per request (a decode step): the whole step from the device's own copy of the slots;
                # rows that pad a captured step carry the spare slot, which no request holds
                slots = ctx.state_slots.long()
                s = self.decay * cache.state[slots] + v
                cache.state[slots] = s
                return s.to(x.dtype)
            out = torch.empty_like(v)
            for r in range(ctx.num_requests):
                slot = ctx.host_state_slots[r]
                s = cache.state[slot].clone()
                for t in range(ctx.host_cu_rows[r], ctx.host_cu_rows[r + 1]):
                    s = self.decay * s + v[t]
                    out[t] = s
                cache.state[slot] = s
            return out.to(x.dtype)

    def build(cfg):
        h = cfg["hidden"]

        def attn(i, window, position):
            p = f"layers.{i}"
            return GroupedQueryAttention(h, cfg["heads"], cfg["kv_heads"], cfg["head_dim"], 1 / math.sqrt(cfg["head_dim"]),
                                         position, AttentionNames(f"{p}.q", f"{p}.k", f"{p}.v", f"{p}.o", f"{p}.qn", f"{p}.kn"),
                                         qk_norm_eps=cfg["eps"], window=window)

        def block(i, mixer):
            p = f"layers.{i}"
            return PreNormBlock(RmsNorm(h, cfg["eps"], f"{p}.n1"), mixer, RmsNorm(h, cfg["eps"], f"{p}.n2"),
                                GatedMlp(h, cfg["inner"], "silu", GatedMlpNames(f"{p}.gate", f"{p}.up", f"{p}.down")))

        rope = lambda: RotaryEncoding(cfg["head_dim"], cfg["theta"])  # noqa: E731
        first = attn(0, cfg["window"] + 6, rope()) if cfg.get("stateless") else DecayingSumMixer(
            h, cfg["decay"], "layers.0.mix", on_device=bool(cfg.get("state_on_device")))
        layers = [block(0, first), block(1, attn(1, None, rope())),
                  block(2, attn(2, cfg["window"], NoPositionEncoding())), block(3, attn(3, None, rope()))]
        # layer 1 runs twice (two caches, one set of weights); layer 3 reads the cache of the first call of layer 1
        program = [LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(1), LayerCall(3, cache_from=1)]
        embedding = TokenEmbedding(cfg["vocab"], h, "embed")
        return DecoderModel(embedding, layers, RmsNorm(h, cfg["eps"], "norm"), OutputHead(cfg["vocab"], h, "head"),
                            vocab_size=cfg["vocab"], max_positions=cfg["max_positions"], program=program)

    register_architecture("ToyHybridForTests", lambda raw: dict(raw.document), build, replace=True)


def plain_toy_forward(cfg, weights, tokens):
    """The toy's whole-sequence reference, from the plain implementation's functions."""
    w = {k: v.double() for k, v in weights.items()}
    n_q, n_kv, d, eps = cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["eps"]
    pos = torch.arange(len(tokens))
    inv = pm.plain_inverse_frequencies(cfg["theta"], d)
    h = w["embed"][torch.tensor(tokens)]
    kept = {}

    def attn(i, x, window, rotate, call, reuse=None):
        p = f"layers.{i}"
        q = pm.plain_rms_norm(pm.plain_linear(x, w[f"{p}.q"]).view(-1, n_q, d), w[f"{p}.qn"], eps)
        if rotate:
            q = pm.plain_rope_neox(q, pos, inv)
        if reuse is None:
            k = pm.plain_rms_norm(pm.plain_linear(x, w[f"{p}.k"]).view(-1, n_kv, d), w[f"{p}.kn"], eps)
            if rotate:
                k = pm.plain_rope_neox(k, pos, inv)
            v = pm.plain_linear(x, w[f"{p}.v"]).view(-1, n_kv, d)
            kept[call] = (k, v)
        else:
            k, v = kept[reuse]
        a = pm.plain_attention(q, k, v, 1 / math.sqrt(d), window=window)
        return pm.plain_linear(a.reshape(len(x), -1), w[f"{p}.o"])

    def mixer0(x):
        v = pm.plain_linear(x, w["layers.0.mix"])
        out, s = [], torch.zeros(cfg["hidden"], dtype=torch.float64)
        for t in range(len(x)):
            s = cfg["decay"] * s + v[t]
            out.append(s)
        return torch.stack(out)

    first = (lambda x: attn(0, x, cfg["window"] + 6, True, 0)) if cfg.get("stateless") else (lambda x: mixer0(x))
    calls = [(0, first), (1, lambda x: attn(1, x, None, True, 1)),
             (2, lambda x: attn(2, x, cfg["window"], False, 2)), (1, lambda x: attn(1, x, None, True, 3)),
             (3, lambda x: attn(3, x, None, True, 4, reuse=1))]
    for layer, mix in calls:
        p = f"layers.{layer}"
        h = h + mix(pm.plain_rms_norm(h, w[f"{p}.n1"], eps))
        n = pm.plain_rms_norm(h, w[f"{p}.n2"], eps)
        h = h + pm.plain_linear(pm.plain_silu_mul(pm.plain_linear(n, w[f"{p}.gate"]), pm.plain_linear(n, w[f"{p}.up"])), w[f"{p}.down"])
    return pm.plain_linear(pm.plain_rms_norm(h, w["norm"], eps), w["head"])


@pytest.mark.parametrize("dtype_name,stored,tolerance", [("float32", torch.float32, rh.FP32_TOLERANCE),
                                                         ("bfloat16", torch.bfloat16, rh.BF16_TOLERANCE)])
def test_an_architecture_defined_in_the_test(tmp_path, dtype_name, stored, tolerance):
    from sglang_rs_b200.cache import CacheManager
    from sglang_rs_b200.config import unregister_architecture
    from sglang_rs_b200.parts import PagedKV, RequestState
    from sglang_rs_b200.weights import read_model_dir, write_model_folder
    register_toy()
    try:
        folder = write_model_folder(str(tmp_path / "toy"), TOY, seed=5, dtype=stored)      # the random-weights mode knows it too
        weights = {k: v.float() for k, v in read_model_dir(folder).items()}
        requests = rh.random_requests({"vocab_size": TOY["vocab"]}, (70, 33, 150, 9, 41), seed=4)
        expected = {rid: plain_toy_forward(TOY, weights, toks).numpy() for rid, toks in requests.items()}
        for make_trace in (rh.trace_whole, rh.trace_portions, lambda r: rh.trace_mixed(r, seed=3)):
            trace = make_trace(requests)
            rows, session = rh.run_in_process(folder, dtype_name, trace)
            bad = rh.first_bad(rows, expected, tolerance)
            print("toy:", rh.worst_error(rows, expected))
            assert bad is None, bad
        needs = session.model.cache_needs()
        assert isinstance(needs[0], RequestState) and needs[4] is None and needs[2] == PagedKV(2, 16, 11)
        assert set(session.cache.allocators) == {("kv", None), ("kv", 11)}
        # generation through the scheduler works for it as well
        from sglang_rs_b200 import Engine
        engine = Engine(model_path=folder, dtype=dtype_name, max_total_tokens=512, chunked_prefill_size=16,
                        max_running_requests=4)
        prompts = [requests["r1"], requests["r3"]]
        results = engine.generate(prompts, {"max_new_tokens": 6})
        for prompt, result in zip(prompts, results):
            tokens = list(prompt)
            for token in result["output_ids"]:
                logits = torch.from_numpy(plain_toy_forward(TOY, weights, tokens).numpy()[-1])
                limit = (0.0 if dtype_name == "float32" else 3e-2) * float(logits.abs().max())
                assert float(logits.max() - logits[token]) <= limit
                tokens.append(token)
    finally:
        unregister_architecture("ToyHybridForTests")


@pytest.mark.parametrize("dtype_name,stored,tolerance", [("float32", torch.float32, rh.FP32_TOLERANCE),
                                                         ("bfloat16", torch.bfloat16, rh.BF16_TOLERANCE)])
def test_a_mixer_with_state_of_its_own_decodes_from_captured_graphs(tmp_path, dtype_name, stored, tolerance):
    """The toy's stateful mixer with its decode step on the device: decode steps are captured (rows that pad a
    captured step use the spare state slot), give the oracle's logits, and in 32-bit the very bits of the
    uncaptured run; portions of prompts still walk their rows in order on the host."""
    from sglang_rs_b200.config import unregister_architecture
    from sglang_rs_b200.weights import read_model_dir, write_model_folder
    toy = dict(TOY, state_on_device=True)
    register_toy()
    try:
        folder = write_model_folder(str(tmp_path / "toy3"), toy, seed=6, dtype=stored)
        weights = {k: v.float() for k, v in read_model_dir(folder).items()}
        requests = rh.random_requests({"vocab_size": TOY["vocab"]}, (70, 33, 150, 9, 41), seed=9)
        expected = {rid: plain_toy_forward(toy, weights, toks).numpy() for rid, toks in requests.items()}
        for trace in (rh.trace_tail_by_one(requests, tail=20), rh.trace_mixed(requests, seed=6, decode_tail=20),
                      rh.trace_decode_together(requests, tail=9)):
            captured, session = rh.run_in_process(folder, dtype_name, trace)
            assert session.runner.graphs is not None and session.runner.graphs.replays >= 9
            assert session.model.native is None                  # a part without a record: the part-by-part path
            bad = rh.first_bad(captured, expected, tolerance)
            assert bad is None, bad
            eager, _ = rh.run_in_process(folder, dtype_name, trace, graphs=False)
            for rid in eager:
                for p, row in eager[rid].items():
                    if dtype_name == "float32":
                        assert np.array_equal(row, captured[rid][p]), (rid, p)
    finally:
        unregister_architecture("ToyHybridForTests")


@pytest.mark.parametrize("dtype_name,stored,tolerance", [("float32", torch.float32, rh.FP32_TOLERANCE),
                                                         ("bfloat16", torch.bfloat16, rh.BF16_TOLERANCE)])
def test_captured_steps_with_window_groups(tmp_path, dtype_name, stored, tolerance):
    """The toy without its stateful mixer is safe to capture: three cache groups (all keys, windows
    of 11 and 17), a layer called twice, a layer that reads another's cache, decoded from CUDA graphs
    and from single launches, with pages of the window groups handed back on the way."""
    from sglang_rs_b200.config import unregister_architecture
    from sglang_rs_b200.weights import read_model_dir, write_model_folder
    toy = dict(TOY, stateless=True)
    register_toy()
    try:
        folder = write_model_folder(str(tmp_path / "toy2"), toy, seed=8, dtype=stored)
        weights = {k: v.float() for k, v in read_model_dir(folder).items()}
        requests = rh.random_requests({"vocab_size": toy["vocab"]}, (90, 45, 200, 33), seed=6)
        expected = {rid: plain_toy_forward(toy, weights, toks).numpy() for rid, toks in requests.items()}
        for trace in (rh.trace_tail_by_one(requests, tail=40), rh.trace_mixed(requests, seed=9, decode_tail=40)):
            for graphs in (False, True):
                rows, session = rh.run_in_process(folder, dtype_name, trace, graphs=graphs)
                assert (session.runner.graphs is not None) == graphs
                if graphs:
                    assert session.runner.graphs.replays > 40
                bad = rh.first_bad(rows, expected, tolerance)
                assert bad is None, (graphs, bad)
        assert set(session.cache.allocators) == {("kv", None), ("kv", 11), ("kv", 17)}
    finally:
        unregister_architecture("ToyHybridForTests")


# ------------------------------------------------------------------------------ more parts defined here
TOY2 = {"architectures": ["ToyPartsForTests"], "hidden": 64, "vocab": 120, "heads": 4, "kv_heads": 4, "head_dim": 16,
        "inner": 48, "eps": 1e-6, "experts": 3, "top_k": 2, "max_positions": 300}


def register_toy_parts():
    """A position encoding whose angles are not position * frequency, and a feed-forward with
    routing, both defined here and used through the framework's interfaces."""
    from sglang_rs_b200 import ops
    from sglang_rs_b200.config import register_architecture
    from sglang_rs_b200.models import DecoderModel
    from sglang_rs_b200.parts import (AttentionNames, FeedForward, GatedMlp, GatedMlpNames, GroupedQueryAttention,
                                      OutputHead, PositionEncoding, PreNormBlock, RmsNorm, TensorSpec, TokenEmbedding,
                                      scale_to)
    from sglang_rs_b200.parts.rope import FusedRotary

    class LogRotary(PositionEncoding):
        """angle(pos, i) = log(1 + pos) * rate[i] + phase[i]; rate and phase are checkpoint tensors."""
        fused = True
        graph_safe = True

        def __init__(self, head_dim, prefix):
            self.head_dim, self.prefix = head_dim, prefix

        def tensor_specs(self):
            return {f"{self.prefix}.rate": TensorSpec((self.head_dim // 2,), "scale"),
                    f"{self.prefix}.phase": TensorSpec((self.head_dim // 2,), "normal")}

        def load(self, tensors, device, dtype):
            self.rate = scale_to(tensors[f"{self.prefix}.rate"], device)
            self.phase = scale_to(tensors[f"{self.prefix}.phase"], device)

        def fused_rotary(self):
            return FusedRotary(None, self.head_dim, False,
                               angles=lambda positions: (torch.log1p(positions.float())[:, None] * self.rate[None, :]
                                                         + self.phase[None, :]).contiguous())

    class RoutedMlp(FeedForward):
        """Router logits in 32-bit, top-k experts, weights = softmax over the chosen logits."""

        def __init__(self, hidden, inner, experts, top_k, prefix):
            self.hidden, self.top_k, self.prefix = hidden, top_k, prefix
            self.experts = [GatedMlp(hidden, inner, "silu", GatedMlpNames(f"{prefix}.e{e}.gate", f"{prefix}.e{e}.up",
                                                                         f"{prefix}.e{e}.down")) for e in range(experts)]

        def tensor_specs(self):
            specs = {f"{self.prefix}.router": TensorSpec((len(self.experts), self.hidden))}
            for expert in self.experts:
                specs.update(expert.tensor_specs())
            return specs

        def load(self, tensors, device, dtype):
            self.router = scale_to(tensors[f"{self.prefix}.router"], device) * 50.0     # clear-cut choices
            for expert in self.experts:
                expert.load(tensors, device, dtype)

        def forward(self, ctx, x):
            logits = x.float() @ self.router.t()
            top, chosen = torch.topk(logits, self.top_k, dim=-1)
            weights = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, expert in enumerate(self.experts):
                rows, slot = torch.nonzero(chosen == e, as_tuple=True)
                if rows.numel():
                    y = expert.forward(ctx, x[rows].contiguous())
                    y = y.sum(0) if y.dim() == 3 else y
                    out.index_add_(0, rows, y.float() * weights[rows, slot][:, None])
            return out.to(x.dtype)

    def build(cfg):
        h, d = cfg["hidden"], cfg["head_dim"]
        layers = []
        for i in range(2):
            p = f"layers.{i}"
            mixer = GroupedQueryAttention(h, cfg["heads"], cfg["kv_heads"], d, 1 / math.sqrt(d), LogRotary(d, f"{p}.pos"),
                                          AttentionNames(f"{p}.q", f"{p}.k", f"{p}.v", f"{p}.o", f"{p}.qn", f"{p}.kn"),
                                          qk_norm_eps=cfg["eps"])
            ffn = RoutedMlp(h, cfg["inner"], cfg["experts"], cfg["top_k"], f"{p}.moe") if cfg["experts"] else \
                GatedMlp(h, cfg["inner"], "silu", GatedMlpNames(f"{p}.gate", f"{p}.up", f"{p}.down"))
            layers.append(PreNormBlock(RmsNorm(h, cfg["eps"], f"{p}.n1"), mixer, RmsNorm(h, cfg["eps"], f"{p}.n2"), ffn))
        embedding = TokenEmbedding(cfg["vocab"], h, "embed")
        return DecoderModel(embedding, layers, RmsNorm(h, cfg["eps"], "norm"), OutputHead(cfg["vocab"], h, None, embedding),
                            vocab_size=cfg["vocab"], max_positions=cfg["max_positions"])

    register_architecture("ToyPartsForTests", lambda raw: dict(raw.document), build, replace=True)


def plain_toy_parts_forward(cfg, weights, tokens):
    w = {k: v.double() for k, v in weights.items()}
    n_q, d, eps = cfg["heads"], cfg["head_dim"], cfg["eps"]
    pos = torch.arange(len(tokens))
    h = w["embed"][torch.tensor(tokens)]

    def rotate(x, p):
        angle = (torch.log1p(pos.float())[:, None] * w[f"{p}.pos.rate"].float()[None, :]
                 + w[f"{p}.pos.phase"].float()[None, :]).double()      # the engine forms the angle in 32-bit
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        a, b = x[..., :d // 2], x[..., d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)

    def gated(x, gate, up, down):
        return pm.plain_linear(pm.plain_silu_mul(pm.plain_linear(x, w[gate]), pm.plain_linear(x, w[up])), w[down])

    for i in range(2):
        p = f"layers.{i}"
        n = pm.plain_rms_norm(h, w[f"{p}.n1"], eps)
        q = rotate(pm.plain_rms_norm(pm.plain_linear(n, w[f"{p}.q"]).view(-1, n_q, d), w[f"{p}.qn"], eps), p)
        k = rotate(pm.plain_rms_norm(pm.plain_linear(n, w[f"{p}.k"]).view(-1, n_q, d), w[f"{p}.kn"], eps), p)
        v = pm.plain_linear(n, w[f"{p}.v"]).view(-1, n_q, d)
        a = pm.plain_attention(q, k, v, 1 / math.sqrt(d))
        h = h + pm.plain_linear(a.reshape(len(tokens), -1), w[f"{p}.o"])
        n = pm.plain_rms_norm(h, w[f"{p}.n2"], eps)
        if cfg["experts"]:
            logits = n @ (w[f"{p}.moe.router"] * 50.0).t()
            top, chosen = torch.topk(logits, cfg["top_k"], dim=-1)
            weights_ = torch.softmax(top, dim=-1)
            out = torch.zeros_like(n)
            for t in range(len(tokens)):
                for j in range(cfg["top_k"]):
                    e = int(chosen[t, j])
                    out[t] += weights_[t, j] * gated(n[t:t + 1], f"{p}.moe.e{e}.gate", f"{p}.moe.e{e}.up", f"{p}.moe.e{e}.down")[0]
            h = h + out
        else:
            h = h + gated(n, f"{p}.gate", f"{p}.up", f"{p}.down")
    return pm.plain_linear(pm.plain_rms_norm(h, w["norm"], eps), w["embed"])


@pytest.mark.parametrize("experts,dtype_name,stored,tolerance", [
    (0, "float32", torch.float32, rh.FP32_TOLERANCE), (0, "bfloat16", torch.bfloat16, rh.BF16_TOLERANCE),
    (3, "float32", torch.float32, rh.FP32_TOLERANCE)])
def test_another_position_encoding_and_a_routed_feed_forward(tmp_path, experts, dtype_name, stored, tolerance):
    """Parts defined in this file: a rotary encoding with logarithmic angles and tensors of its
    own (it hands the fused kernel an angle per row and pair), and a feed-forward that routes each
    row to 2 of 3 experts (32-bit router; tested in 32-bit, where a close call cannot fall the
    other way).  Decoded steps of the first run from CUDA graphs."""
    from sglang_rs_b200.config import unregister_architecture
    from sglang_rs_b200.weights import read_model_dir, write_model_folder
    toy = dict(TOY2, experts=experts)
    register_toy_parts()
    try:
        folder = write_model_folder(str(tmp_path / "parts"), toy, seed=3, dtype=stored)
        weights = {k: v.float() for k, v in read_model_dir(folder).items()}
        requests = rh.random_requests({"vocab_size": toy["vocab"]}, (70, 33, 150, 9), seed=2)
        expected = {rid: plain_toy_parts_forward(toy, weights, toks).numpy() for rid, toks in requests.items()}
        for trace in (rh.trace_whole(requests), rh.trace_tail_by_one(requests), rh.trace_mixed(requests, seed=6)):
            rows, session = rh.run_in_process(folder, dtype_name, trace)
            bad = rh.first_bad(rows, expected, tolerance)
            print("toy parts:", rh.worst_error(rows, expected))
            assert bad is None, bad
        assert (session.runner.graphs is not None) == (experts == 0)
    finally:
        unregister_architecture("ToyPartsForTests")


def test_step_records_kernel_classes_and_request_totals(tmp_path):
    """What the engine counts: a record per step (rows, kinds of rows, pages free, host and device time), the
    device time per kernel class when tracing is on, and the totals over requests in the reference's names."""
    from sglang_rs_b200 import Engine
    from sglang_rs_b200.ops import trace
    folder = rh.make_folder(tmp_path, "m", pm.TINY_D, seed=3, dtype=torch.bfloat16)
    engine = Engine(model_path=folder, dtype="bfloat16", max_total_tokens=1024, chunked_prefill_size=32,
                    disable_cuda_graph=True)
    prompts = list(rh.random_requests(pm.TINY_D, (70, 9, 33), seed=8).values())
    saved = trace.active
    try:
        trace.configure("events")
        results = engine.generate(prompts, {"max_new_tokens": 5, "ignore_eos": True})
    finally:
        trace.active = saved
    records = engine.runner.step_log.flush()
    assert len(records) == engine.runner.steps_run and records[-1] is engine.runner.last_stats
    assert sum(r.prompt_rows + r.decode_rows for r in records) == sum(r.rows for r in records)
    assert sum(r.rows for r in records) == sum(len(p) for p in prompts) + 3 * 4      # the last token is never fed
    assert all(r.rows <= 32 + 3 for r in records) and any(r.decode_rows and r.prompt_rows for r in records)
    assert all(r.device_ms is not None and r.device_ms > 0 and r.host_ms > 0 for r in records)
    kinds = set().union(*(r.kernels for r in records))
    assert {"embedding", "norm", "gemm", "rope_kv"} <= kinds and any(k.startswith("attention") for k in kinds)
    for r in records:
        assert 0 < sum(r.kernels.values()) <= r.device_ms * 1.05 + 0.05
    assert "kv:None" in records[0].pages_free
    m = engine.metrics
    assert (m.requests_total, m.requests_in_flight, m.requests_failed_total) == (3, 0, 0)
    assert m.prompt_tokens_total == sum(len(p) for p in prompts) and m.generation_tokens_total == 15
    assert m.time_to_first_token_seconds_count == 3 and m.request_duration_seconds_count == 3
    assert all(len(r["output_ids"]) == 5 for r in results)
    assert "sglang_generation_tokens_total 15" in m.render()


def test_tokens_stream_through_a_sink_and_a_sink_can_end_a_request(tmp_path):
    """``generate(..., sink=...)``: every step's output reaches the sink as soon as it is on the host; a sink that
    returns False ends that request alone (the reference's rule, crates/sglang-srt/src/engine.rs:294-297).  The other
    requests produce what they produce without a sink, and the ended request's pages are given back."""
    from sglang_rs_b200 import Engine
    folder = rh.make_folder(tmp_path, "m", pm.TINY_A, seed=4, dtype=torch.float32)
    prompts = list(rh.random_requests(pm.TINY_A, (21, 40, 9), seed=2).values())
    params = {"max_new_tokens": 12, "ignore_eos": True}
    plain = Engine(model_path=folder, dtype="float32", max_total_tokens=512, chunked_prefill_size=16).generate(prompts, params)
    engine = Engine(model_path=folder, dtype="float32", max_total_tokens=512, chunked_prefill_size=16,
                    disable_radix_cache=True)
    seen = {0: [], 1: [], 2: []}
    finished = {}

    def sink(index, output):
        seen[index].extend(output.token_ids)
        if output.finished:
            finished[index] = output.finish_reason
        return not (index == 1 and len(seen[1]) >= 3)          # the second request is ended after three tokens

    results = engine.generate(prompts, params, sink=sink)
    assert [r["output_ids"] for r in results] == [seen[0], seen[1], seen[2]]
    assert results[0]["output_ids"] == plain[0]["output_ids"] and results[2]["output_ids"] == plain[2]["output_ids"]
    assert 3 <= len(seen[1]) <= 4 and seen[1] == plain[1]["output_ids"][:len(seen[1])]     # a step was in flight
    assert results[1]["finish_reason"] == "abort" and finished == {0: "length", 1: "abort", 2: "length"}
    assert not engine.scheduler.has_work and engine._in_flight is None
    engine.cache.check_invariants()
    assert all(a.free_count == a.num_pages for a in engine.cache.allocators.values())
    assert engine.metrics.requests_failed_total == 1 and engine.metrics.requests_in_flight == 0
