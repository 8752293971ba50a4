"""Configuration and registry (no GPU)."""
import json

import pytest

from plain_model import TINY_A, TINY_B, TINY_C
from sglang_rs_b200.config import (ConfigError, RawConfig, register_architecture,
                                   registered_architectures, resolve_architecture, unregister_architecture)
from sglang_rs_b200 import models  # noqa: F401
from sglang_rs_b200.models.qwen3_config import Qwen3Config


def parse(document):
    return Qwen3Config.from_raw(RawConfig.from_dict(document))


def test_tiny_configs_parse_and_differ_everywhere():
    a, b, c = parse(TINY_A), parse(TINY_B), parse(TINY_C)
    for field in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "max_position_embeddings",
                  "tie_word_embeddings"):
        assert getattr(a, field) != getattr(b, field), field
    assert c.attention_bias and not a.attention_bias
    assert b.num_attention_heads * b.head_dim != b.hidden_size


def test_defaults_follow_the_reference():
    doc = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta",
                                                        "max_position_embeddings", "tie_word_embeddings")}
    cfg = parse(doc)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rope_theta == 1_000_000.0 and cfg.max_position_embeddings == 32768
    assert cfg.tie_word_embeddings is False          # tied only if literally true


def test_rope_theta_from_rope_parameters_and_text_config_nesting():
    doc = dict(TINY_A)
    del doc["rope_theta"]
    doc["rope_parameters"] = {"rope_type": "default", "rope_theta": 5000.0}
    assert parse(doc).rope_theta == 5000.0
    nested = {"architectures": ["Qwen3ForCausalLM"], "text_config": {k: v for k, v in TINY_B.items() if k != "architectures"}}
    assert parse(nested).hidden_size == TINY_B["hidden_size"]


@pytest.mark.parametrize("change, fragment", [
    ({"hidden_act": None}, "hidden_act"),
    ({"hidden_act": "gelu"}, "unsupported hidden_act"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"vocab_size": 0}, "non-zero"),
    ({"num_hidden_layers": None}, "num_hidden_layers"),
    ({"num_key_value_heads": 3}, "divisible"),
    ({"head_dim": 15}, "even head_dim"),
    ({"use_sliding_window": True, "sliding_window": 128}, "sliding-window"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "RoPE variant yarn"),
    ({"rope_scaling": {"type": "default", "mrope_section": [1, 2]}}, "RoPE variant"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"rms_norm_eps": -1e-6}, "rms_norm_eps"),
    ({"max_position_embeddings": 0}, "max_position_embeddings"),
])
def test_rejections(change, fragment):
    doc = dict(TINY_A)
    for key, value in change.items():
        if value is None:
            doc.pop(key, None)
        else:
            doc[key] = value
    with pytest.raises(ConfigError) as error:
        parse(doc)
    assert fragment in str(error.value)


@pytest.mark.parametrize("change, fragment", [
    ({"head_dim": 520}, "head_dim 520 is outside what the attention kernels take"),
    ({"num_attention_heads": 66, "num_key_value_heads": 2, "head_dim": 16}, "33 query heads per kv head exceed"),
])
def test_sizes_that_the_kernels_refuse_are_refused_when_the_model_is_built(change, fragment):
    """config.json may hold them (the reference asks only for an even head_dim, models/qwen.rs:129-157); the
    kernels do not take them, and the error comes at load with the keys' names, not at the first step."""
    from sglang_rs_b200.weights import build_model
    with pytest.raises(ConfigError) as error:
        build_model(dict(TINY_A, **change))
    assert fragment in str(error.value) and "head_dim=" in str(error.value) and "Qwen3ForCausalLM" in str(error.value)
    # an even head_dim that is no multiple of 16 is taken
    model, config = build_model(dict(TINY_A, head_dim=18))
    assert config.head_dim == 18


def test_head_dim_must_divide_when_derived():
    doc = dict(TINY_A, hidden_size=66)
    del doc["head_dim"]
    with pytest.raises(ConfigError, match="divisible by attention head divisor"):
        parse(doc)


def test_eos_ids_int_or_list():
    assert RawConfig.from_dict(dict(TINY_A, eos_token_id=7)).eos_token_ids == (7,)
    assert RawConfig.from_dict(dict(TINY_A, eos_token_id=[7, 9])).eos_token_ids == (7, 9)
    assert parse(dict(TINY_A, eos_token_id=[7, 9])).eos_token_ids == (7, 9)


def test_round_trip_document():
    cfg = parse(TINY_C)
    again = parse(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


def test_registry_resolves_first_known_and_lists_supported():
    entry = resolve_architecture(RawConfig.from_dict({"architectures": ["Nope", "Qwen3ForCausalLM"]}))
    assert entry.name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="missing `architectures`"):
        resolve_architecture(RawConfig.from_dict({}))
    with pytest.raises(ConfigError) as error:
        resolve_architecture(RawConfig.from_dict({"architectures": ["LlamaForCausalLM"]}))
    assert "Qwen3ForCausalLM" in str(error.value) and "LlamaForCausalLM" in str(error.value)


def test_registering_another_architecture_needs_no_framework_change():
    register_architecture("ToyForTests", lambda raw: {"n": raw.document["n"]}, lambda cfg: ("model", cfg["n"]))
    try:
        assert "ToyForTests" in registered_architectures()
        entry = resolve_architecture(RawConfig.from_dict({"architectures": ["ToyForTests"], "n": 3}))
        assert entry.build_model(entry.parse_config(RawConfig.from_dict({"architectures": ["ToyForTests"], "n": 3}))) == ("model", 3)
        with pytest.raises(ValueError):
            register_architecture("ToyForTests", None, None)
    finally:
        unregister_architecture("ToyForTests")


def test_model_sizes_come_from_config_only():
    from sglang_rs_b200.weights import build_model
    for doc in (TINY_A, TINY_B, TINY_C):
        model, cfg = build_model(doc)
        specs = model.tensor_specs()
        assert specs["model.embed_tokens.weight"].shape == (cfg.vocab_size, cfg.hidden_size)
        assert ("lm_head.weight" in specs) == (not cfg.tie_word_embeddings)
        q = specs["model.layers.0.self_attn.q_proj.weight"].shape
        assert q == (cfg.num_attention_heads * cfg.head_dim, cfg.hidden_size)
        assert specs["model.layers.0.self_attn.k_norm.weight"].shape == (cfg.head_dim,)
        assert ("model.layers.0.self_attn.o_proj.bias" in specs) == cfg.attention_bias
        assert len(model.layers) == cfg.num_hidden_layers
