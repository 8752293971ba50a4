"""The plain implementation against hand-derived anchors, vectors of the reference's own tests and its own
invariants (no GPU)."""
import json
import os

import pytest
import torch

import plain_model as pm

ANCHORS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "plain_anchors.json")))
T = lambda v: torch.tensor(v, dtype=torch.float64)  # noqa: E731


def test_rms_norm_anchor():
    a = ANCHORS["rms_norm"]
    assert torch.allclose(pm.plain_rms_norm(T(a["x"]), T(a["w"]), a["eps"]), T(a["y"]), atol=1e-12)


def test_linear_anchor():
    a = ANCHORS["linear"]
    assert torch.equal(pm.plain_linear(T(a["x"]), T(a["w"]), T(a["b"])), T(a["y"]))


def test_rope_anchor_and_theta_table():
    a = ANCHORS["rope_neox"]
    inv = pm.plain_inverse_frequencies(a["theta"], 4)
    out = pm.plain_rope_neox(T(a["x"]).view(1, 1, 4), torch.tensor([a["position"]]), inv)
    assert torch.allclose(out.view(-1), T(a["y"]), atol=1e-7)
    inv = pm.plain_inverse_frequencies(10000.0, 8)
    assert torch.allclose(inv.double(), T([1.0, 0.1, 0.01, 0.001]), rtol=1e-6)
    unchanged = pm.plain_rope_neox(T(a["x"]).view(1, 1, 4), torch.tensor([0]), inv[:2])
    assert torch.equal(unchanged.view(-1), T(a["x"]))


def test_silu_mul_anchor():
    a = ANCHORS["silu_mul"]
    assert torch.allclose(pm.plain_silu_mul(T(a["g"]), T(a["u"])), T(a["y"]), atol=1e-12)


def test_attention_anchor_and_grouping():
    a = ANCHORS["attention"]
    q = T([a["q"], a["q"]]).view(2, 1, 2)
    out = pm.plain_attention(q, T(a["k"]).view(2, 1, 2), T(a["v"]).view(2, 1, 2), a["scale"])
    assert torch.allclose(out[0, 0], T(a["y_first"])) and torch.allclose(out[1, 0], T(a["y_last"]), atol=1e-12)
    # consecutive query heads share a kv head
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 4, 8).double(), torch.randn(3, 2, 8).double(), torch.randn(3, 2, 8).double()
    out = pm.plain_attention(q, k, v, 0.3)
    alone = pm.plain_attention(q[:, 2:3], k[:, 1:2], v[:, 1:2], 0.3)
    assert torch.allclose(out[:, 2:3], alone)
    # a window of 2 at the last position sees only the last two keys
    windowed = pm.plain_attention(q, k, v, 0.3, window=2)
    tail = pm.plain_attention(q[2:3], k[1:3], v[1:3], 0.3, first_position=1)
    assert torch.allclose(windowed[2], tail[0]) and torch.allclose(windowed[:2], out[:2])


def test_vectors_of_the_reference_tests():
    """Inputs and expected outputs copied as data from the reference's own kernel tests
    (crates/sglang-kernel/tests/cpu_kernels.rs:63-80, :174-190, :200-238)."""
    a = ANCHORS["gqa_one_token"]
    q = T(a["q"]).view(1, a["query_heads"], a["head_dim"])
    k, v = T(a["k"]).view(1, a["kv_heads"], a["head_dim"]), T(a["v"]).view(1, a["kv_heads"], a["head_dim"])
    assert torch.equal(pm.plain_attention(q, k, v, a["scale"]).reshape(-1), T(a["y"]))
    a = ANCHORS["rope_partial"]
    x = T(a["x"]).view(1, 1, 6)
    got = pm.plain_rope_neox(x, torch.tensor([a["position"]]), pm.plain_inverse_frequencies(a["theta"], a["rotary_dim"]))
    assert torch.allclose(got.reshape(-1), T(a["y"]), atol=1e-7)
    a = ANCHORS["top_k_renorm"]
    for row, (probs, fixed, k_row, per_row) in enumerate(zip(a["probs"], a["fixed_y"], a["per_row_k"], a["per_row_y"])):
        logits = torch.log(T(probs))
        for k, want in ((a["fixed_k"], fixed), (k_row, per_row)):
            kept = pm.plain_filtered_distribution(logits, 1.0, top_k=k, top_p=None, min_p=None)
            total = sum(kept.values())
            got = [kept.get(i, 0.0) / total for i in range(len(probs))]
            assert max(abs(g - w) for g, w in zip(got, want)) < 1e-12, (row, k, got, want)


def one_hot_model():
    config = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 3, "num_hidden_layers": 1, "hidden_size": 4,
              "intermediate_size": 4, "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 2,
              "hidden_act": "silu", "attention_bias": False, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
              "max_position_embeddings": 32, "tie_word_embeddings": False}
    z = torch.zeros
    p = "model.layers.0"
    weights = {
        "model.embed_tokens.weight": torch.tensor([[0., 0, 0, 0], [1, 0, 0, 0], [0, 1, 0, 0]]),
        "model.norm.weight": torch.ones(4),
        "lm_head.weight": torch.tensor([[0., 0, 0, 0], [0, 1, 0, 0], [1, 0, 0, 0]]),
        f"{p}.self_attn.q_proj.weight": z(4, 4), f"{p}.self_attn.k_proj.weight": z(2, 4),
        f"{p}.self_attn.v_proj.weight": z(2, 4), f"{p}.self_attn.o_proj.weight": z(4, 4),
        f"{p}.self_attn.q_norm.weight": torch.ones(2), f"{p}.self_attn.k_norm.weight": torch.ones(2),
        f"{p}.input_layernorm.weight": torch.ones(4), f"{p}.post_attention_layernorm.weight": torch.ones(4),
        f"{p}.mlp.gate_proj.weight": z(4, 4), f"{p}.mlp.up_proj.weight": z(4, 4), f"{p}.mlp.down_proj.weight": z(4, 4),
    }
    return config, weights


def test_one_hot_model_of_the_reference():
    config, weights = one_hot_model()
    a = ANCHORS["one_hot_model"]
    assert pm.plain_greedy(config, weights, a["prompt"], len(a["greedy"])) == a["greedy"]


@pytest.mark.parametrize("config", [pm.TINY_A, pm.TINY_B, pm.TINY_C])
def test_causality_and_precision(config):
    weights = pm.plain_random_weights(config, seed=5)
    tokens = torch.randint(0, config["vocab_size"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = pm.plain_forward(config, weights, tokens)
    assert whole.shape == (23, config["vocab_size"]) and whole.dtype == torch.float64
    prefix = pm.plain_forward(config, weights, tokens[:9])
    assert torch.allclose(whole[:9], prefix, atol=1e-12)            # later tokens change nothing earlier
    single = pm.plain_forward(config, weights, tokens, dtype=torch.float32)
    scale = float(whole.abs().max())
    assert float((single.double() - whole).abs().max()) < 1e-5 * scale


def test_sampling_helpers():
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0])
    assert pm.plain_argmax(logits) == 1
    p = torch.softmax(logits.double() / 0.7, 0)
    edges = torch.cumsum(p, 0)
    for u, want in ((0.0, 0), (float(edges[0]) + 1e-9, 1), (float(edges[1]) + 1e-9, 2), (0.999999, 3 if float(edges[2]) < 0.999999 else 2)):
        assert pm.plain_temperature_sample(logits, 0.7, u) == want
    kept = pm.plain_filtered_distribution(logits, 1.0, top_k=3, top_p=None, min_p=None)
    assert set(kept) == {0, 1, 2}
    kept = pm.plain_filtered_distribution(logits, 1.0, top_k=None, top_p=0.5, min_p=None)
    assert set(kept) == {1, 2}                                     # mass before the second item is still < 0.5
    kept = pm.plain_filtered_distribution(logits, 1.0, top_k=None, top_p=None, min_p=0.5)
    assert set(kept) == {1, 2}
    out = pm.plain_apply_penalties(torch.tensor([2.0, -2.0, 1.0]), [0, 0, 1], frequency=0.5, presence=0.25, repetition=2.0)
    assert torch.allclose(out, torch.tensor([2.0 / 2 - 0.25 - 1.0, -2.0 * 2 - 0.25 - 0.5, 1.0]))
