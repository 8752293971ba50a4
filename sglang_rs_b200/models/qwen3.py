"""Qwen3 dense (``Qwen3ForCausalLM``) put together from the parts.

Checkpoint names as the reference binds them (crates/sglang-srt/src/models/qwen.rs:321-353):
``model.embed_tokens.weight``, ``model.norm.weight``, ``lm_head.weight`` unless tied, and per
layer ``input_layernorm``, ``self_attn.{q,k,v,o}_proj`` (+ ``.bias`` with ``attention_bias``),
``self_attn.{q,k}_norm``, ``post_attention_layernorm``, ``mlp.{gate,up,down}_proj``.
Fixed by the architecture, not by config.json: half-split rotary over the whole head,
scale 1/sqrt(head_dim), the same eps for all norms (crates/sglang-srt/src/cpu_reference.rs:
278-299, :493-536).
"""
from __future__ import annotations

import math

from ..config.model_config import ConfigError
from ..config.registry import register_architecture
from ..parts import (AttentionNames, GatedMlp, GatedMlpNames, GroupedQueryAttention, OutputHead, PreNormBlock,
                     RmsNorm, RotaryEncoding, TokenEmbedding)
from .decoder import DecoderModel
from .qwen3_config import Qwen3Config


def build_qwen3(config: Qwen3Config) -> DecoderModel:
    """Sizes that config.json may hold and that a part refuses (a head wider than the attention kernels
    take, too many query heads per kv head) are reported here, at load, under the architecture's name."""
    try:
        return _build(config)
    except ValueError as error:
        if isinstance(error, ConfigError):
            raise
        raise ConfigError(
            Qwen3Config.ARCHITECTURE,
            f"{error} (head_dim={config.head_dim}, num_attention_heads={config.num_attention_heads}, "
            f"num_key_value_heads={config.num_key_value_heads})") from None


def _build(config: Qwen3Config) -> DecoderModel:
    embedding = TokenEmbedding(config.vocab_size, config.hidden_size, "model.embed_tokens.weight")
    # one encoding for all layers: its table of frequencies is a constant of the model, and layers that share it
    # share, within a step, the cosines and sines computed from it
    rotary = RotaryEncoding(config.head_dim, config.rope_theta)
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}"
        bias = (lambda name: f"{prefix}.self_attn.{name}_proj.bias") if config.attention_bias else (lambda name: None)
        names = AttentionNames(
            q=f"{prefix}.self_attn.q_proj.weight", k=f"{prefix}.self_attn.k_proj.weight",
            v=f"{prefix}.self_attn.v_proj.weight", o=f"{prefix}.self_attn.o_proj.weight",
            q_norm=f"{prefix}.self_attn.q_norm.weight", k_norm=f"{prefix}.self_attn.k_norm.weight",
            q_bias=bias("q"), k_bias=bias("k"), v_bias=bias("v"), o_bias=bias("o"))
        mixer = GroupedQueryAttention(
            config.hidden_size, config.num_attention_heads, config.num_key_value_heads, config.head_dim,
            scale=1.0 / math.sqrt(config.head_dim),
            position=rotary,
            names=names, qk_norm_eps=config.rms_norm_eps, window=None)
        feed_forward = GatedMlp(
            config.hidden_size, config.intermediate_size, config.hidden_act,
            GatedMlpNames(gate=f"{prefix}.mlp.gate_proj.weight", up=f"{prefix}.mlp.up_proj.weight",
                          down=f"{prefix}.mlp.down_proj.weight"))
        layers.append(PreNormBlock(
            RmsNorm(config.hidden_size, config.rms_norm_eps, f"{prefix}.input_layernorm.weight"), mixer,
            RmsNorm(config.hidden_size, config.rms_norm_eps, f"{prefix}.post_attention_layernorm.weight"),
            feed_forward))
    final_norm = RmsNorm(config.hidden_size, config.rms_norm_eps, "model.norm.weight")
    head = OutputHead(config.vocab_size, config.hidden_size,
                      None if config.tie_word_embeddings else "lm_head.weight", embedding)
    # exporters of this architecture may store the rotation's frequency table, and a head beside a tied
    # embedding; the reference binds by name and reads neither (crates/sglang-srt/src/models/qwen.rs:321-353)
    ignored = ["*.rotary_emb.inv_freq"] + (["lm_head.weight"] if config.tie_word_embeddings else [])
    return DecoderModel(embedding, layers, final_norm, head, vocab_size=config.vocab_size,
                        max_positions=config.max_position_embeddings, eos_token_ids=config.eos_token_ids,
                        ignored_tensors=ignored)


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_raw, build_qwen3, replace=True)
