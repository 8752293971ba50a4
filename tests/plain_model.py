"""A plain, slow implementation of Qwen3 dense: whole sequences, no cache, one function for
each part.  It shares no code with the engine (it has its own reader for safetensors and
reads config.json keys itself) and is the oracle of every numeric test.

It rests on the formulas of the reference's host code, cited per function as
``file:line`` inside ``crates/``.  The reference is a Rust workspace and neither ``cargo``
nor ``rustc`` exists on this machine, so its own model code cannot be compiled or run here
for a one-time cross-check; ``tests/golden/`` therefore holds only hand-derived anchors (see
``tests/golden/make_golden.py``).

Arithmetic is float64 by default (``dtype``), so that the difference between an engine run
and this oracle is the engine's own rounding.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ----------------------------------------------------------------------------- files
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Independent minimal reader: 8-byte length, JSON header, payload
    (sglang-srt/src/model_artifacts.rs:1456-1514)."""
    with open(path, "rb") as handle:
        (length,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(length))
        payload = handle.read()
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        raw = np.frombuffer(payload[begin:end], dtype=np.uint8).copy()
        kind = entry["dtype"]
        if kind == "F32":
            tensor = torch.from_numpy(raw.view(np.float32).copy())
        elif kind == "BF16":       # bf16 = upper half of an f32 (model_artifacts.rs:917-961)
            wide = raw.view(np.uint16).astype(np.uint32) << 16
            tensor = torch.from_numpy(wide.view(np.float32).copy())
        elif kind == "F16":
            tensor = torch.from_numpy(raw.view(np.float16).astype(np.float32))
        else:
            raise ValueError(f"plain reader: dtype {kind} of {name}")
        out[name] = tensor.reshape(entry["shape"])
    return out


def load_folder(folder: str):
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


def round_to_bf16(tensor: torch.Tensor) -> torch.Tensor:
    """Round to nearest even to bfloat16 and widen again
    (sglang-srt/src/cuda_transformer.rs:537-546)."""
    return tensor.to(torch.float32).to(torch.bfloat16).to(torch.float32)


# ----------------------------------------------------------------------------- parts
def plain_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y_i = x_i / sqrt(mean(x^2) + eps) * w_i over the last axis
    (sglang-kernel/src/cpu.rs:26-34)."""
    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x / torch.sqrt(mean_square + eps) * weight


def plain_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[o] = sum_i x[i] W[o, i] (+ b[o]); W is [out, in] (sglang-kernel/src/cpu.rs:73-108)."""
    y = x @ weight.t()
    return y if bias is None else y + bias


def plain_silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """g / (1 + exp(-g)) * u (sglang-kernel/src/cpu.rs:119-123)."""
    return gate / (1.0 + torch.exp(-gate)) * up


def plain_inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """theta^(-2i/rotary_dim) in 64-bit, then cast to 32-bit (sglang-kernel/src/rotary.rs:72-98)."""
    values = [float(theta) ** (-2.0 * i / rotary_dim) for i in range(rotary_dim // 2)]
    return torch.tensor(values, dtype=torch.float64).to(torch.float32)


def plain_rope_neox(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of [tokens, heads, d]: pairs (i, i + d/2), angle = float32(pos) *
    inv_freq[i] taken in 32-bit, then (a cos - b sin, b cos + a sin)
    (sglang-kernel/src/rotary.rs:216-236)."""
    half = inv_freq.numel()
    angle = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(x.dtype)   # 32-bit product
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:2 * half]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = b * cos + a * sin
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: Optional[int] = None, first_position: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of a whole sequence.  q [T, n_q, d]; k, v [S, n_kv, d]
    with S = first_position + T.  kv head = q head // (n_q / n_kv); s = (q . k) * scale over
    keys 0..pos (or the last ``window`` of them); softmax with the maximum subtracted;
    weighted sum of v (sglang-kernel/src/cpu.rs:475-517; keys by length,
    sglang-srt/src/cpu_reference.rs:161)."""
    tokens, n_q, d = q.shape
    n_kv = k.shape[1]
    group = n_q // n_kv
    out = torch.zeros_like(q)
    for t in range(tokens):
        pos = first_position + t
        lo = 0 if window is None else max(0, pos - window + 1)
        for head in range(n_q):
            kv_head = head // group
            scores = (k[lo:pos + 1, kv_head] @ q[t, head]) * scale
            weights = torch.exp(scores - scores.max())
            weights = weights / weights.sum()
            out[t, head] = weights @ v[lo:pos + 1, kv_head]
    return out


def plain_attention_block(x, weights, prefix, config, positions, dtype):
    """Attention half of a layer (sglang-srt/src/cpu_reference.rs:442-546): projections,
    per-head q/k norm before the rotation (:487-506), rotation (:507-524), attention with
    scale 1/sqrt(d) (:536), output projection (:545)."""
    n_q, n_kv = config["num_attention_heads"], config.get("num_key_value_heads") or config["num_attention_heads"]
    d = config.get("head_dim") or config["hidden_size"] // n_q
    eps = config["rms_norm_eps"]
    bias = (lambda name: weights[f"{prefix}.self_attn.{name}_proj.bias"]) if config.get("attention_bias") \
        else (lambda name: None)
    q = plain_linear(x, weights[f"{prefix}.self_attn.q_proj.weight"], bias("q")).view(-1, n_q, d)
    k = plain_linear(x, weights[f"{prefix}.self_attn.k_proj.weight"], bias("k")).view(-1, n_kv, d)
    v = plain_linear(x, weights[f"{prefix}.self_attn.v_proj.weight"], bias("v")).view(-1, n_kv, d)
    q = plain_rms_norm(q, weights[f"{prefix}.self_attn.q_norm.weight"], eps)
    k = plain_rms_norm(k, weights[f"{prefix}.self_attn.k_norm.weight"], eps)
    inv_freq = plain_inverse_frequencies(config.get("rope_theta", 1_000_000.0), d)
    q, k = plain_rope_neox(q, positions, inv_freq), plain_rope_neox(k, positions, inv_freq)
    attended = plain_attention(q, k, v, 1.0 / math.sqrt(d))
    return plain_linear(attended.reshape(-1, n_q * d), weights[f"{prefix}.self_attn.o_proj.weight"], bias("o"))


def plain_mlp_block(x, weights, prefix):
    """SwiGLU feed-forward (sglang-srt/src/cpu_reference.rs:585-603)."""
    gate = plain_linear(x, weights[f"{prefix}.mlp.gate_proj.weight"])
    up = plain_linear(x, weights[f"{prefix}.mlp.up_proj.weight"])
    return plain_linear(plain_silu_mul(gate, up), weights[f"{prefix}.mlp.down_proj.weight"])


def plain_forward(config: dict, weights: Dict[str, torch.Tensor], token_ids: Sequence[int],
                  dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence (sglang-srt/src/cpu_reference.rs:123-187 for the
    stack, :257-317 for a layer): embedding row, then per layer h += attn(norm(h)),
    h += mlp(norm(h)), final norm, head (lm_head, or the embedding when tied is literally
    true: sglang-srt/src/models/qwen.rs:225)."""
    w = {name: tensor.to(dtype) for name, tensor in weights.items()}
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    positions = torch.arange(len(ids))
    eps = config["rms_norm_eps"]
    h = w["model.embed_tokens.weight"][ids]
    for layer in range(config["num_hidden_layers"]):
        prefix = f"model.layers.{layer}"
        normed = plain_rms_norm(h, w[f"{prefix}.input_layernorm.weight"], eps)
        h = h + plain_attention_block(normed, w, prefix, config, positions, dtype)
        normed = plain_rms_norm(h, w[f"{prefix}.post_attention_layernorm.weight"], eps)
        h = h + plain_mlp_block(normed, w, prefix)
    normed = plain_rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") is True else w["lm_head.weight"]
    return plain_linear(normed, head)


# ----------------------------------------------------------------------------- sampling
def plain_argmax(logits: torch.Tensor) -> int:
    """Index of the largest logit, the lowest index among equals (the reference's
    ``max_by`` keeps the last of equal maxima, sglang-srt/src/model_executor.rs:592-599; the
    engine documents the lowest)."""
    return int(torch.argmax(logits).item())


def plain_temperature_sample(logits: torch.Tensor, temperature: float, u: float) -> int:
    """p_i = exp(l_i/T - max l/T); the first index, in vocabulary order, whose running sum
    exceeds u * sum(p) (sglang-srt/src/model_executor.rs:471-480, :532-555, walking the
    vocabulary in index order instead of sorted order)."""
    scaled = logits.to(torch.float64) / temperature
    p = torch.exp(scaled - scaled.max())
    running = torch.cumsum(p, dim=0)
    target = u * float(p.sum())
    hits = torch.nonzero(running > target)
    return int(hits[0].item()) if len(hits) else int(torch.nonzero(p > 0)[-1].item())


def plain_filtered_distribution(logits: torch.Tensor, temperature: float, top_k: Optional[int],
                                top_p: Optional[float], min_p: Optional[float]) -> Dict[int, float]:
    """Token -> unnormalised probability after top-k, top-p and min-p
    (sglang-srt/src/model_executor.rs:483-522): sort descending, keep k, keep an item while the
    mass before it is < top_p, drop items below max_p * min_p."""
    scaled = logits.to(torch.float64) / temperature
    p = torch.exp(scaled - scaled.max())
    order = sorted(range(len(p)), key=lambda i: -float(p[i]))
    if top_k is not None and 0 < top_k < len(order):
        order = order[:top_k]
    total = sum(float(p[i]) for i in order)
    floor = float(p[order[0]]) * (min_p or 0.0)
    kept, before = {}, 0.0
    for i in order:
        keep = before < (1.0 if top_p is None else top_p)
        before += float(p[i]) / total
        if keep and float(p[i]) >= floor:
            kept[i] = float(p[i])
    return kept


def plain_apply_penalties(logits: torch.Tensor, seen: Sequence[int], frequency: float, presence: float,
                          repetition: float) -> torch.Tensor:
    """Penalties on tokens of prompt + output (sglang-srt/src/model_executor.rs:558-590)."""
    out = logits.clone()
    counts: Dict[int, int] = {}
    for token in seen:
        counts[token] = counts.get(token, 0) + 1
    for token, count in counts.items():
        if token >= len(out):
            continue
        if repetition != 1.0:
            out[token] = out[token] * repetition if out[token] < 0 else out[token] / repetition
        out[token] -= presence
        out[token] -= frequency * count
    return out


def plain_greedy(config: dict, weights: Dict[str, torch.Tensor], prompt: Sequence[int], steps: int,
                 dtype: torch.dtype = torch.float64) -> List[int]:
    tokens = list(prompt)
    for _ in range(steps):
        tokens.append(plain_argmax(plain_forward(config, weights, tokens, dtype)[-1]))
    return tokens[len(prompt):]


# ----------------------------------------------------------------------------- test models
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 256, "hidden_act": "silu", "attention_bias": False,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 224,
    "vocab_size": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    "max_position_embeddings": 128, "hidden_act": "silu", "attention_bias": False,
}
# a third one with sizes that are no power of two anywhere, biases, one kv head, long enough for page reuse
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 72,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 200,
    "vocab_size": 331, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 640, "hidden_act": "silu", "attention_bias": True,
}


# head_dim 128 and 64: the sizes the tensor-core attention kernels take (A, B and C run the generic one)
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 256,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 640,
    "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 1024, "hidden_act": "silu", "attention_bias": False,
}
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 192,
    "num_attention_heads": 6, "num_key_value_heads": 6, "head_dim": 64, "intermediate_size": 320,
    "vocab_size": 777, "rope_theta": 20000.0, "rms_norm_eps": 2e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 512, "hidden_act": "silu", "attention_bias": True,
}
# an even head_dim that is no multiple of 16 (the reference asks only for an even one, models/qwen.rs:129-157)
TINY_F = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 88,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 18, "intermediate_size": 136,
    "vocab_size": 300, "rope_theta": 30000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 320, "hidden_act": "silu", "attention_bias": False,
}


def plain_random_weights(config: dict, seed: int) -> Dict[str, torch.Tensor]:
    """Own initialiser (not the engine's): N(0, 0.02) matrices, norms 1 + U(-0.1, 0.1)."""
    gen = torch.Generator().manual_seed(seed)
    n_q = config["num_attention_heads"]
    n_kv = config.get("num_key_value_heads") or n_q
    d = config.get("head_dim") or config["hidden_size"] // n_q
    hidden, inner, vocab = config["hidden_size"], config["intermediate_size"], config["vocab_size"]

    def matrix(*shape):
        return torch.randn(*shape, generator=gen) * 0.02

    def scale(width):
        return 1.0 + (torch.rand(width, generator=gen) * 2 - 1) * 0.1

    weights = {"model.embed_tokens.weight": matrix(vocab, hidden), "model.norm.weight": scale(hidden)}
    if config.get("tie_word_embeddings") is not True:
        weights["lm_head.weight"] = matrix(vocab, hidden)
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}"
        weights[f"{p}.input_layernorm.weight"] = scale(hidden)
        weights[f"{p}.post_attention_layernorm.weight"] = scale(hidden)
        weights[f"{p}.self_attn.q_proj.weight"] = matrix(n_q * d, hidden)
        weights[f"{p}.self_attn.k_proj.weight"] = matrix(n_kv * d, hidden)
        weights[f"{p}.self_attn.v_proj.weight"] = matrix(n_kv * d, hidden)
        weights[f"{p}.self_attn.o_proj.weight"] = matrix(hidden, n_q * d)
        weights[f"{p}.self_attn.q_norm.weight"] = scale(d)
        weights[f"{p}.self_attn.k_norm.weight"] = scale(d)
        if config.get("attention_bias"):
            weights[f"{p}.self_attn.q_proj.bias"] = matrix(n_q * d)
            weights[f"{p}.self_attn.k_proj.bias"] = matrix(n_kv * d)
            weights[f"{p}.self_attn.v_proj.bias"] = matrix(n_kv * d)
            weights[f"{p}.self_attn.o_proj.bias"] = matrix(hidden)
        weights[f"{p}.mlp.gate_proj.weight"] = matrix(inner, hidden)
        weights[f"{p}.mlp.up_proj.weight"] = matrix(inner, hidden)
        weights[f"{p}.mlp.down_proj.weight"] = matrix(hidden, inner)
    return weights
