"""Attention mixer over the paged cache: grouped-query, causal, optional window,
optional per-head q/k norm, optional rotation.

One fused projection q|k|v (the reference also stores the three matrices as one,
pegainfer-qwen3/src/weights/load.rs:98-134), then the fused norm + rotation + cache
write, attention over the request's pages, and the output projection
(pegainfer-qwen3/src/unified_forward.rs:414-536). When the call reads another call's
cache only the query projection exists and nothing is written.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import KvNeed
from ..kernels import attention as attn_kernels
from ..kernels.linear import linear
from .base import CacheBinding, Mixer
from .registry import build_position_encoding, register_mixer
from .spec import AttentionSpec, ParamInfo


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: AttentionSpec) -> None:
        super().__init__(spec)
        s = spec
        if s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads ({s.num_heads}) must be a multiple of num_kv_heads ({s.num_kv_heads})")
        if s.head_dim % 8 or s.head_dim > 256:
            raise ValueError(f"head_dim {s.head_dim} unsupported: multiples of 8 up to 256")
        self.q_dim = s.num_heads * s.head_dim
        self.kv_dim = s.num_kv_heads * s.head_dim
        self.position = build_position_encoding(s.position)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm_w: Optional[torch.Tensor] = None
        self.k_norm_w: Optional[torch.Tensor] = None
        self.tables = None

    def kv_need(self) -> Optional[KvNeed]:
        s = self.spec
        return KvNeed(s.num_kv_heads, s.head_dim, s.window)

    def parameters(self) -> Dict[str, ParamInfo]:
        s = self.spec
        p = {
            "q_proj.weight": ParamInfo((self.q_dim, s.hidden_size)),
            "k_proj.weight": ParamInfo((self.kv_dim, s.hidden_size)),
            "v_proj.weight": ParamInfo((self.kv_dim, s.hidden_size)),
            "o_proj.weight": ParamInfo((s.hidden_size, self.q_dim)),
        }
        if s.qk_norm is not None:
            p["q_norm.weight"] = ParamInfo((s.head_dim,), ("one_plus_normal", 0.02))
            p["k_norm.weight"] = ParamInfo((s.head_dim,), ("one_plus_normal", 0.02))
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        q, k, v = tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("q_proj, k_proj and v_proj must be stored in one dtype to be fused")
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.spec.qk_norm is not None:
            self.q_norm_w = tensors["q_norm.weight"].contiguous()
            self.k_norm_w = tensors["k_norm.weight"].contiguous()
            if self.q_norm_w.dtype != self.k_norm_w.dtype:
                self.k_norm_w = self.k_norm_w.to(self.q_norm_w.dtype)

    def prepare(self, device: torch.device, dtype: torch.dtype) -> None:
        self.tables = self.position.rotation_tables(device)

    def forward(self, x: torch.Tensor, ctx, binding: CacheBinding) -> torch.Tensor:
        s = self.spec
        if binding.kv is None:
            raise RuntimeError("attention needs a cache binding")
        group = ctx.groups[binding.kv.group]
        k_cache, v_cache, page_stride = ctx.cache.kv_views(binding.kv)
        w = self.w_qkv if binding.owns_kv else self.w_qkv[: self.q_dim]
        qkv = linear(x, w)
        cos, sin = self.tables if self.tables is not None else (None, None)
        qn = s.qk_norm
        out = torch.empty((x.shape[0], self.q_dim), dtype=x.dtype, device=x.device)
        # One native call: the norm + rotation + cache write (in a kernel of its own, or inside the decode kernel when
        # the step is single tokens in one wave), then the attention kernel(s) that take the step's shape.
        step = attn_kernels.attention_step(ctx, group, qkv, out, k_cache, page_stride, s.num_heads, s.num_kv_heads,
                                           s.head_dim, s.window, cos=cos, q_norm_w=self.q_norm_w)
        layer = attn_kernels.attention_layer(
            qkv, out, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim, s.softmax_scale, s.window,
            q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, eps=qn.eps if qn else 0.0,
            weight_offset=qn.weight_offset if qn else 0.0, cos=cos, sin=sin, write_kv=binding.owns_kv, rope_mode=1,
            interleaved=bool(getattr(s.position, "interleaved", False)))
        attn_kernels.run_attention(step, layer)
        return linear(out, self.w_o)
