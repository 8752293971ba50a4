"""Safetensors reading, binding by name, load errors and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from plain_model import TINY_A, TINY_B, load_folder, read_safetensors
from sglang_rs_b200.weights import (SafetensorsError, WeightLoadError, build_model, load_checkpoint, read_file,
                                    read_model_dir, stored_form, write_file, write_model_folder)


def test_round_trip_all_dtypes(tmp_path):
    tensors = {
        "a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.randn(2, 2).to(torch.float16),
        "d": torch.arange(6, dtype=torch.int64).reshape(2, 3), "e": torch.tensor(3.5), "f": torch.zeros(0, 4),
    }
    path = str(tmp_path / "x.safetensors")
    write_file(path, tensors, {"k": "v"})
    back = read_file(path)
    assert set(back) == set(tensors)
    for name, tensor in tensors.items():
        assert back[name].dtype == tensor.dtype and back[name].shape == tensor.shape
        assert torch.equal(back[name], tensor)
    # the independent reader of the plain implementation agrees on the float tensors
    floats = str(tmp_path / "floats.safetensors")
    write_file(floats, {name: tensors[name] for name in "abc"})
    plain = read_safetensors(floats)
    assert torch.equal(plain["a"], tensors["a"]) and torch.equal(plain["b"], tensors["b"].float())
    assert torch.equal(plain["c"], tensors["c"].float())


def test_stored_form_rule():
    # float16 is kept as stored: the 32-bit path widens it exactly, the bfloat16 path rounds it once
    assert stored_form(torch.zeros(2, dtype=torch.float16)).dtype == torch.float16
    assert stored_form(torch.zeros(2, dtype=torch.bfloat16)).dtype == torch.bfloat16
    assert stored_form(torch.zeros(2, dtype=torch.float32)).dtype == torch.float32      # 32-bit stays 32-bit
    assert stored_form(torch.zeros(2, dtype=torch.int64)).dtype == torch.int32          # integer tables
    assert stored_form(torch.zeros(2, dtype=torch.float64)).dtype == torch.float32


def test_header_faults(tmp_path):
    path = str(tmp_path / "bad.safetensors")
    with open(path, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        read_file(path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds the file"):
        read_file(path)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="do not match shape"):
        read_file(path)
    header = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the payload"):
        read_file(path)
    header = json.dumps({"t": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 2]}}).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + b"\0" * 2)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        read_file(path)


def test_model_folder_and_one_error_for_everything(tmp_path):
    folder = write_model_folder(str(tmp_path / "m"), TINY_B, seed=3, dtype=torch.float32)
    model, _ = build_model(folder)
    expected = {name: spec.shape for name, spec in model.tensor_specs().items()}
    good = load_checkpoint(folder, expected)
    assert set(good) == set(expected)

    tensors = dict(read_model_dir(folder))
    del tensors["model.layers.1.mlp.down_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.ones(5)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.ones(4, 4)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)
    tensors["model.layers.0.self_attn.extra.weight"] = torch.ones(16)
    write_file(os.path.join(folder, "model.safetensors"), tensors)
    with pytest.raises(WeightLoadError) as error:
        load_checkpoint(folder, expected)
    e = error.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.down_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.extra.weight", "model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert [name for name, _, _ in e.wrong_shape] == ["model.layers.0.self_attn.q_norm.weight",
                                                      "model.layers.2.self_attn.k_proj.weight"]
    text = str(e)
    for fragment in ("missing tensors (2)", "unexpected tensors (2)", "wrong shapes (2)", "expected [32] found [5]"):
        assert fragment in text


def test_buffers_that_exporters_write_are_not_an_error(tmp_path):
    """A tied model whose file also holds ``lm_head.weight``, and rotary frequency buffers: the model names
    them as ignorable, so they load (the reference binds by name and never reads them); any other
    unexpected tensor is still an error."""
    folder = write_model_folder(str(tmp_path / "tied"), TINY_A, seed=5, dtype=torch.float32)
    model, _ = build_model(folder)
    expected = {name: spec.shape for name, spec in model.tensor_specs().items()}
    tensors = dict(read_model_dir(folder))
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(8)
    write_file(os.path.join(folder, "model.safetensors"), tensors)
    good = load_checkpoint(folder, expected, model.ignored_tensors)
    assert set(good) == set(expected) and "lm_head.weight" not in good
    with pytest.raises(WeightLoadError) as error:
        load_checkpoint(folder, expected)                    # without the model's list both are unexpected
    assert error.value.unexpected == ["lm_head.weight", "model.layers.1.self_attn.rotary_emb.inv_freq"]
    # an untied model does not ignore a head: there it is expected, and a second one under another name is not
    untied, _ = build_model(write_model_folder(str(tmp_path / "untied"), TINY_B, seed=5, dtype=torch.float32))
    assert "lm_head.weight" not in untied.ignored_tensors and "lm_head.weight" in untied.tensor_specs()


def test_float16_checkpoint_is_widened_exactly_for_the_32_bit_path(tmp_path):
    """The host side of the rule: a float16 tensor reaches the part unrounded, and the part's cast to
    float32 is exact (the reference widens every stored float type, model_artifacts.rs:850-860)."""
    from sglang_rs_b200.parts.base import matrix_to, scale_to
    folder = write_model_folder(str(tmp_path / "h"), TINY_A, seed=9, dtype=torch.float16)
    model, _ = build_model(folder)
    loaded = load_checkpoint(folder, {name: spec.shape for name, spec in model.tensor_specs().items()},
                             model.ignored_tensors)
    _, plain = load_folder(folder)                           # the plain reader widens float16 exactly
    for name, tensor in loaded.items():
        assert tensor.dtype == torch.float16
        assert torch.equal(matrix_to(tensor, "cpu", torch.float32), plain[name])
        assert torch.equal(scale_to(tensor, "cpu"), plain[name])
    # values that bfloat16 cannot hold survive
    assert any(not torch.equal(t.float(), t.to(torch.bfloat16).float()) for t in loaded.values())


def test_sharded_folder_with_index(tmp_path):
    folder = str(tmp_path / "s")
    os.makedirs(folder)
    write_file(os.path.join(folder, "model-00001-of-00002.safetensors"), {"a": torch.ones(2)})
    write_file(os.path.join(folder, "model-00002-of-00002.safetensors"), {"b": torch.zeros(3)})
    with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {"a": "model-00001-of-00002.safetensors", "b": "model-00002-of-00002.safetensors"}}, f)
    assert set(read_model_dir(folder)) == {"a", "b"}
    os.remove(os.path.join(folder, "model-00002-of-00002.safetensors"))
    with pytest.raises(SafetensorsError, match="does not exist"):
        read_model_dir(folder)


def test_random_weights_statistics_and_determinism(tmp_path):
    one = write_model_folder(str(tmp_path / "one"), TINY_A, seed=11, dtype=torch.float32)
    two = write_model_folder(str(tmp_path / "two"), TINY_A, seed=11, dtype=torch.float32)
    other = write_model_folder(str(tmp_path / "other"), TINY_A, seed=12, dtype=torch.float32)
    a, b, c = read_model_dir(one), read_model_dir(two), read_model_dir(other)
    assert all(torch.equal(a[name], b[name]) for name in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    embed = a["model.embed_tokens.weight"]
    assert abs(float(embed.std()) - 0.02) < 0.002 and abs(float(embed.mean())) < 0.002
    norm = a["model.layers.0.input_layernorm.weight"]
    assert float(norm.min()) >= 0.9 and float(norm.max()) <= 1.1 and float(norm.std()) > 0.01
    assert "lm_head.weight" not in a                          # tiny A ties its head
    config, plain = load_folder(one)
    assert config == TINY_A and torch.equal(plain["model.norm.weight"], a["model.norm.weight"])
    bf = read_model_dir(write_model_folder(str(tmp_path / "bf"), TINY_A, seed=11, dtype=torch.bfloat16))
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert torch.equal(bf["model.embed_tokens.weight"], embed.to(torch.bfloat16))
