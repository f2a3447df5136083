"""Qwen3 dense (``Qwen3ForCausalLM``) configuration.

Keys and defaults follow the reference's serde struct
(pegainfer-qwen3/src/config.rs:27-44): ``head_dim`` is a key of its own
(independent of hidden_size / num_attention_heads), ``max_position_embeddings``
defaults to 40960 (config.rs:166-168), and keys the reference does not read
(attention_bias, hidden_act, rope_scaling, sliding_window, ...) are ignored.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

from .base import ConfigError, ModelConfig


@dataclasses.dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int = 40960
    # The reference requires eos_token_id; a random-weights folder has no
    # tokenizer, so here it may be absent (nothing then stops generation early).
    eos_token_id: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self) -> None:
        for key in (
            "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings",
        ):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{key} must be positive, got {getattr(self, key)}")
        # pegainfer-qwen3/src/config.rs:196-204
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be a positive multiple "
                f"of num_key_value_heads ({self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim ({self.head_dim}) must be even for rotate-half RoPE")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")

    def with_stop_token_ids(self, ids) -> "Qwen3Config":
        return dataclasses.replace(self, stop_token_ids=tuple(int(i) for i in ids))

    def to_dict(self):
        d = super().to_dict()
        d.pop("stop_token_ids", None)
        if d.get("eos_token_id") is None:
            d.pop("eos_token_id", None)
        return d

    # derived sizes
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim
