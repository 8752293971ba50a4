"""Validated configuration of a ``Qwen3ForCausalLM`` checkpoint (the architecture's own keys).

It lives beside the architecture's builder (``models/qwen3.py``); the shared configuration module holds
only what every architecture uses: the raw document and the readers of typed keys.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

from ..config.model_config import (ConfigError, RawConfig, missing_field, optional_bool, optional_float,
                                   optional_positive_int, required_positive_int)


@dataclass(frozen=True)
class Qwen3Config:
    """Validated fields of a ``Qwen3ForCausalLM`` checkpoint.

    Keys, defaults and rejections are the reference adapter's
    (``crates/sglang-srt/src/models/qwen.rs:104-244``): ``num_key_value_heads``
    defaults to the query head count and must divide it (``:120-128``);
    ``head_dim`` defaults to ``hidden_size / num_attention_heads`` and must be even
    (``:129-157``); ``hidden_act`` must be ``"silu"`` (``:159-170``); a sliding
    window is rejected (``:171-179``); only default RoPE is accepted (``:254-289``);
    ``rms_norm_eps`` has no default (``:182-191``); ``rope_theta`` defaults to 1e6
    and may sit in ``rope_parameters`` (``:192-195``); ``max_position_embeddings``
    defaults to 32768 (``:202``); embeddings are tied only if the key is literally
    true (``:225``).
    """

    ARCHITECTURE = "Qwen3ForCausalLM"

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    hidden_act: str
    eos_token_ids: Sequence[int] = ()
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_raw(cls, raw: RawConfig) -> "Qwen3Config":
        arch = cls.ARCHITECTURE
        doc = raw.text
        vocab_size = required_positive_int(arch, doc, "vocab_size")
        num_layers = required_positive_int(arch, doc, "num_hidden_layers")
        hidden_size = required_positive_int(arch, doc, "hidden_size")
        intermediate_size = required_positive_int(arch, doc, "intermediate_size")
        num_heads = required_positive_int(arch, doc, "num_attention_heads")
        num_kv_heads = doc.get("num_key_value_heads")
        if num_kv_heads is None:
            num_kv_heads = num_heads
        if isinstance(num_kv_heads, bool) or not isinstance(num_kv_heads, int) or num_kv_heads <= 0 \
                or num_heads % num_kv_heads != 0:
            raise ConfigError(
                arch,
                f"num_attention_heads ({num_heads}) must be divisible by non-zero "
                f"num_key_value_heads ({num_kv_heads})",
            )
        original_heads = optional_positive_int(arch, doc, "original_num_attention_heads")
        head_dim = doc.get("head_dim")
        if original_heads is not None or head_dim is None:
            divisor = original_heads if original_heads is not None else num_heads
            if hidden_size % divisor != 0:
                raise ConfigError(
                    arch, f"hidden_size ({hidden_size}) must be divisible by attention head divisor ({divisor})"
                )
            head_dim = hidden_size // divisor
        else:
            if isinstance(head_dim, bool) or not isinstance(head_dim, int):
                raise ConfigError(arch, f"`head_dim` must be an integer, found {head_dim!r}")
            if head_dim <= 0:
                raise ConfigError(arch, "head_dim must be non-zero")
        if head_dim % 2 != 0:
            raise ConfigError(arch, f"NeoX RoPE requires an even head_dim, found {head_dim}")

        hidden_act = doc.get("hidden_act")
        if hidden_act is None:
            raise missing_field(arch, "hidden_act")
        if hidden_act != "silu":
            raise ConfigError(arch, f"unsupported hidden_act {hidden_act}; the dense decoder requires silu")
        if optional_bool(arch, doc, "use_sliding_window") is True:
            raise ConfigError(
                arch, f"sliding-window attention is not implemented (sliding_window={doc.get('sliding_window')!r})"
            )
        _validate_default_rope(arch, doc)

        eps = optional_float(arch, doc, "rms_norm_eps")
        if eps is None:
            raise missing_field(arch, "rms_norm_eps")
        if not math.isfinite(eps) or eps < 0.0:
            raise ConfigError(arch, "rms_norm_eps must be finite and non-negative")
        theta = optional_float(arch, doc, "rope_theta")
        if theta is None:
            params = doc.get("rope_parameters")
            if isinstance(params, dict) and isinstance(params.get("rope_theta"), (int, float)):
                theta = float(params["rope_theta"])
        if theta is None:
            theta = 1_000_000.0
        if not math.isfinite(theta) or theta <= 0.0:
            raise ConfigError(arch, "rope_theta must be finite and positive")
        max_pos = doc.get("max_position_embeddings")
        if max_pos is None:
            max_pos = 32_768
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
            raise ConfigError(arch, "max_position_embeddings must be non-zero")

        return cls(
            vocab_size=vocab_size,
            hidden_size=hidden_size,
            intermediate_size=intermediate_size,
            num_hidden_layers=num_layers,
            num_attention_heads=num_heads,
            num_key_value_heads=num_kv_heads,
            head_dim=head_dim,
            rms_norm_eps=eps,
            rope_theta=theta,
            max_position_embeddings=max_pos,
            tie_word_embeddings=optional_bool(arch, doc, "tie_word_embeddings") is True,
            attention_bias=optional_bool(arch, doc, "attention_bias") is True,
            hidden_act=hidden_act,
            eos_token_ids=tuple(raw.eos_token_ids),
            raw=dict(raw.document),
        )

    def to_dict(self) -> dict[str, Any]:
        """A ``config.json`` document that parses back to this configuration."""
        document: dict[str, Any] = {
            "architectures": [self.ARCHITECTURE],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "use_sliding_window": False,
        }
        if self.eos_token_ids:
            ids = list(self.eos_token_ids)
            document["eos_token_id"] = ids[0] if len(ids) == 1 else ids
        return document


def _validate_default_rope(architecture: str, doc: Mapping[str, Any]) -> None:
    scaling = doc.get("rope_scaling")
    if scaling is None:
        scaling = doc.get("rope_parameters")
    if scaling is None:
        return
    if not isinstance(scaling, dict):
        raise ConfigError(architecture, "rope_scaling/rope_parameters must be an object")
    rope_type = scaling.get("rope_type", scaling.get("type", "default"))
    if not isinstance(rope_type, str):
        rope_type = "default"
    if rope_type != "default" or "mrope_section" in scaling or scaling.get("use_fope") is True:
        raise ConfigError(architecture, f"RoPE variant {rope_type} is not implemented by the dense decoder")
