"""Qwen3 dense: how a ``Qwen3Config`` becomes a ``ModelSpec``.

Every layer is the same pre-norm block: RMSNorm -> grouped-query attention with
per-head q/k RMSNorm (same eps as the layer norms) and full-head rotate-half RoPE ->
residual, RMSNorm -> SwiGLU -> residual; final RMSNorm; head tied to the embedding or
``lm_head.weight`` (pegainfer-qwen3/src/weights/load.rs:84-206, config.rs:223-229,
unified_forward.rs:383-611). softmax scale 1/sqrt(head_dim), no window
(pegainfer-kernels/src/ops/attention.rs:507; csrc/shared/paged_attention.cu:560-566).
Tensor names are the checkpoint's own (weights/load.rs:84-206).
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.qwen3 import Qwen3Config
from ..parts.spec import AttentionSpec, BlockSpec, GatedMlpSpec, ModelSpec, NormSpec, PositionSpec


def build_spec(cfg: Qwen3Config) -> ModelSpec:
    layer_norm = NormSpec(kind="rms", size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    head_norm = NormSpec(kind="rms", size=cfg.head_dim, eps=cfg.rms_norm_eps)
    position = PositionSpec(kind="rope", rotary_dim=cfg.head_dim, theta=cfg.rope_theta,
                            max_positions=cfg.max_position_embeddings)
    mixer = AttentionSpec(
        hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
        num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
        softmax_scale=1.0 / math.sqrt(cfg.head_dim), position=position, qk_norm=head_norm, window=None)
    ffn = GatedMlpSpec(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, activation="silu")
    blocks = tuple(
        BlockSpec(kind="prenorm", name=f"model.layers.{i}.", mixer=mixer, feed_forward=ffn,
                  input_norm=layer_norm, post_norm=layer_norm,
                  mixer_name="self_attn.", feed_forward_name="mlp.",
                  input_norm_name="input_layernorm.", post_norm_name="post_attention_layernorm.")
        for i in range(cfg.num_hidden_layers))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, blocks=blocks,
        order=tuple(range(cfg.num_hidden_layers)), final_norm=layer_norm,
        embedding_name="model.embed_tokens.weight", final_norm_name="model.norm.",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings, stop_token_ids=tuple(cfg.stop_token_ids))


register_architecture(Qwen3Config.architecture, Qwen3Config, build_spec)
