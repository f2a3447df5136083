"""The bfloat16 twin of the plain implementation: the same formulas with the REFERENCE's rounding points.

The reference stores every activation in bfloat16 between operations and rounds inside some of them; this
file restates where (each function cites the lines): the per-head q/k norm rounds twice, the rotation rounds
every product and then the sum, its cos/sin table is bfloat16, SiLU is rounded before it is multiplied by `up`,
each residual sum is rounded and the norm behind it reads the rounded sum, the logits are bfloat16. Products
take bfloat16 operands and add up in float32 (here: float32 matrix products of bfloat16-valued tensors).

The engine does NOT reproduce these roundings: its kernels round once per output (one rounding in the q/k norm,
float32 rotation tables, the activation rounded once, float32 logits). So the engine's bfloat16 logits are not
equal to this twin's element by element; what the tests check with it is that the engine is at least as close
to the float32 plain implementation as the reference's own scheme of rounding would be, and that the two
bfloat16 computations agree within the bfloat16 tolerance. It rests on the reference's formulas (the reference
itself cannot be compiled here), imports nothing from the package, and shares the unrounded pieces with
``plain_qwen3``.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

import plain_qwen3 as plain


def bf(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 (nearest even) and widen again: the value a bfloat16 tensor would hold."""
    return x.to(torch.bfloat16).to(torch.float32)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Sum of squares and scale in float32, ONE rounding (pegainfer-kernels/csrc/shared/flashinfer_norm.cu:204-210)."""
    return bf(plain.rms_norm(x, weight, eps))


def head_norm(u: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head q/k norm with TWO roundings: n = bf16(u * rsqrt(mean(u^2) + eps)), then bf16(n * w)
    (pegainfer-kernels/csrc/shared/prefill_attention.cu:84-99)."""
    n = bf(u * torch.rsqrt((u * u).mean(dim=-1, keepdim=True) + eps))
    return bf(n * weight)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half with a bfloat16 table and a rounding after every product and after the sum:
    out[d] = bf16(bf16(x[d] cos) - bf16(x[d + half] sin)) for d < half, bf16(bf16(x[d - half] sin) + bf16(x[d] cos))
    beyond (pegainfer-core/src/weight_loader.rs:730-764; prefill_attention.cu:101-122). x is [T, heads, head_dim]."""
    hd = x.shape[-1]
    cos, sin = plain.rope_tables(hd, theta, positions)
    c, s = bf(cos)[:, None, :], bf(sin)[:, None, :]
    lo, hi = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([bf(bf(lo * c) - bf(hi * s)), bf(bf(lo * s) + bf(hi * c))], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Scores and softmax in float32 from bfloat16 q and k; the probabilities are rounded to bfloat16 for the
    second product, whose sum is float32 and whose result is rounded once
    (pegainfer-kernels/csrc/shared/paged_attention.cu:439-567: the library's tensor-core kernel)."""
    T, nq, hd = q.shape
    group = nq // k.shape[1]
    out = torch.zeros_like(q)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    for h in range(nq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].t()) * scale
        s = s.masked_fill(j > i, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        out[:, h, :] = (bf(p) @ v[:, kh, :]) / p.sum(dim=-1, keepdim=True)
    return bf(out)


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, positions: torch.Tensor) -> torch.Tensor:
    """pegainfer-qwen3/src/prefill.rs:206-316; every projection's output is stored in bfloat16."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = bf(plain.linear(x, w[prefix + "q_proj.weight"])).view(T, nq, hd)
    k = bf(plain.linear(x, w[prefix + "k_proj.weight"])).view(T, nkv, hd)
    v = bf(plain.linear(x, w[prefix + "v_proj.weight"])).view(T, nkv, hd)
    q = apply_rope(head_norm(q, w[prefix + "q_norm.weight"], eps), positions, cfg["rope_theta"])
    k = apply_rope(head_norm(k, w[prefix + "k_norm.weight"], eps), positions, cfg["rope_theta"])
    o = causal_attention(q, k, v, 1.0 / math.sqrt(hd))
    return bf(plain.linear(o.reshape(T, nq * hd), w[prefix + "o_proj.weight"]))


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """act = bf16(f32(bf16(silu(g))) * f32(u)): SiLU is rounded BEFORE the multiply
    (pegainfer-kernels/csrc/shared/elementwise.cu:259-273; pegainfer-qwen3/src/unified_forward.rs:557-595)."""
    g = bf(plain.linear(x, w[prefix + "gate_proj.weight"]))
    u = bf(plain.linear(x, w[prefix + "up_proj.weight"]))
    act = bf(bf(g / (1.0 + torch.exp(-g))) * u)
    return bf(plain.linear(act, w[prefix + "down_proj.weight"]))


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], token_ids: List[int]) -> torch.Tensor:
    """Logits [T, vocab] as the reference's bfloat16 path would round them: h = bf16(h + branch) after each branch,
    the norm reads the rounded sum (flashinfer_norm.cu:76-83, 107-124), logits stored in bfloat16
    (pegainfer-qwen3/src/prefill.rs:440-477). ``w``: the folder's tensors widened to float32 (they are bfloat16 values)."""
    positions = torch.arange(len(token_ids))
    h = plain.embedding(torch.tensor(token_ids, dtype=torch.long), w["model.embed_tokens.weight"])
    eps = cfg["rms_norm_eps"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        a = attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, positions)
        h = bf(h + a)
        m = swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
        h = bf(h + m)
    h = rms_norm(h, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return bf(plain.linear(h, head))
