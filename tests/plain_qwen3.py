"""Plain, slow 32-bit implementation of the Qwen3 dense decoder: the tests' oracle.

It rests on the reference's FORMULAS, not on its code running here: the
reference (a Rust + CUDA workspace) cannot be compiled or imported on a CPU box
without a Rust toolchain, its Qwen3 kernels need FlashInfer headers that are not
in its tree, and they reject the tiny shapes used in the tests (head_dim must be
128, pegainfer-kernels/csrc/shared/prefill_attention.cu:310). So nothing under
tests/golden/ comes from the reference; every function below cites the lines
whose arithmetic it restates, in float32 throughout (the reference rounds to
bf16 between ops; this oracle does not).

Whole sequences, no cache, one function per part, plain loops where a loop is
the clearest statement. Shares no code with the package (it does not import
``openinfer_b200``); it reads config.json and model.safetensors by itself.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch
from safetensors import safe_open


# --------------------------------------------------------------------------
# loading
# --------------------------------------------------------------------------
def read_model_folder(folder: str, dtype: torch.dtype = torch.float32):
    """config.json as a dict and every tensor of model.safetensors widened to float32 (or, for an
    oracle whose own rounding is out of the picture at real layer widths, to float64: every function
    below computes in the type of the tensors it is given; rotation angles stay float32 by definition)."""
    with open(os.path.join(folder, "config.json")) as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt", device="cpu") as f:
        for name in f.keys():
            tensors[name] = f.get_tensor(name).to(dtype)
    return cfg, tensors


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t,:] = embed_tokens[ids[t],:], a copy without scaling
    (pegainfer-kernels/csrc/shared/elementwise.cu:368-384; pegainfer-qwen3/src/prefill.rs:144-165)."""
    return table[ids.long()].clone()


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis; the weight is used as it is,
    no (1 + w) (pegainfer-kernels/csrc/shared/flashinfer_norm.cu:170-187, 204-210)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = W x without bias; W is stored [out, in] row-major
    (pegainfer-kernels/csrc/shared/linear.cu:312-362; pegainfer-qwen3/src/unified_forward.rs:414-453)."""
    return x @ weight.t()


def rope_tables(head_dim: int, theta: float, positions: torch.Tensor):
    """inv_freq[i] = 1 / theta^(2i/head_dim), angle = pos * inv_freq[i], all float32
    (pegainfer-core/src/weight_loader.rs:730-764)."""
    half = head_dim // 2
    idx = torch.arange(half, dtype=torch.float32)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float32), idx * 2.0 / head_dim)
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    return torch.cos(ang), torch.sin(ang)  # [T, half]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half over the full head: for d < half, out[d] = x[d]*cos - x[d+half]*sin;
    for d >= half, out[d] = x[d-half]*sin + x[d]*cos
    (pegainfer-kernels/csrc/shared/prefill_attention.cu:101-122). x is [T, heads, head_dim]."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, lo * s + hi * c], dim=-1)


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None
) -> torch.Tensor:
    """s[i,j] = (q_i . k_j) * scale for j <= i, softmax over j, o_i = sum_j p[i,j] v_j;
    query head h reads kv head h // (nq / nkv); scale = 1/sqrt(head_dim), no soft-cap, no sinks
    (pegainfer-kernels/csrc/shared/paged_attention.cu:439-567; pegainfer-kernels/src/ops/attention.rs:507).
    ``window`` (not used by Qwen3: the reference passes window_left = -1) keeps only the last
    ``window`` keys, the query's own position included.
    q [T, nq, hd], k/v [T, nkv, hd] -> [T, nq, hd]."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.zeros_like(q)
    for h in range(nq):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].t()) * scale  # [T, T]
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        mask = j <= i
        if window is not None:
            mask = mask & (j > i - window)
        scores = scores.masked_fill(~mask, float("-inf"))
        p = torch.softmax(scores, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_block(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict,
                    positions: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Projections, per-head q/k RMSNorm (before RoPE, same eps as the layer norms; v untouched),
    RoPE, causal GQA attention, output projection
    (pegainfer-qwen3/src/prefill.rs:206-316; prefill_attention.cu:84-99)."""
    T = x.shape[0]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    eps = cfg["rms_norm_eps"]
    q = linear(x, w[prefix + "q_proj.weight"]).view(T, nq, hd)
    k = linear(x, w[prefix + "k_proj.weight"]).view(T, nkv, hd)
    v = linear(x, w[prefix + "v_proj.weight"]).view(T, nkv, hd)
    q = rms_norm(q, w[prefix + "q_norm.weight"], eps)
    k = rms_norm(k, w[prefix + "k_norm.weight"], eps)
    cos, sin = rope_tables(hd, cfg["rope_theta"], positions)
    q = apply_rope(q, cos, sin)
    k = apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(hd), window)
    return linear(o.reshape(T, nq * hd), w[prefix + "o_proj.weight"])


def swiglu(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down( silu(gate x) * (up x) ), silu(g) = g / (1 + exp(-g))
    (pegainfer-qwen3/src/unified_forward.rs:557-595; elementwise.cu:259-273)."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    act = g / (1.0 + torch.exp(-g)) * u
    return linear(act, w[prefix + "down_proj.weight"])


def decoder_layer(h: torch.Tensor, w: Dict[str, torch.Tensor], i: int, cfg: dict,
                  positions: torch.Tensor) -> torch.Tensor:
    """Pre-norm block with two residuals (pegainfer-qwen3/src/unified_forward.rs:383-611)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    a = attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.", cfg, positions)
    h = h + a
    m = swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    return h + m


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], token_ids: List[int]) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence
    (embedding -> layers -> final norm -> head; the head is embed_tokens when
    tie_word_embeddings, else lm_head: pegainfer-qwen3/src/config.rs:223-229, prefill.rs:440-477)."""
    ids = torch.tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(token_ids))
    h = embedding(ids, w["model.embed_tokens.weight"])
    for i in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, i, cfg, positions)
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(h, head)


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """n argmax tokens, lowest index on ties (pegainfer-kernels/csrc/shared/argmax.cu:15-18),
    recomputing the whole sequence each time."""
    seq = list(prompt)
    out: List[int] = []
    for _ in range(n):
        logits = forward_logits(cfg, w, seq)[-1]
        tok = int(torch.argmax(logits).item())
        out.append(tok)
        seq.append(tok)
    return out


# --------------------------------------------------------------------------
# sampling (plain restatement of the parameter semantics)
# --------------------------------------------------------------------------
def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int = -1,
                          top_p: float = 1.0, min_p: float = 0.0) -> torch.Tensor:
    """The distribution a sampled token is drawn from: softmax(logits / T), then top-k,
    then top-p on the renormalised rest, then min-p relative to the largest probability
    (order of the reference's pipeline, pegainfer-kernels/csrc/shared/flashinfer_sampling.cu:99-128;
    parameter meanings pegainfer-frontend/src/sampler.rs:2-38). Ties at a threshold are kept.
    Computed in float64 on a float32 softmax input."""
    p = torch.softmax(logits.to(torch.float32) / temperature, dim=-1).to(torch.float64)
    V = p.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        q = torch.where(keep, p, torch.zeros_like(p))
        q = q / q.sum()
        vals, _ = torch.sort(q, descending=True)
        csum = torch.cumsum(vals, 0)
        n = int((csum < top_p).sum().item()) + 1  # smallest prefix reaching top_p
        thr = vals[min(n, V) - 1]
        keep &= q >= thr
    if min_p > 0.0:
        keep &= p >= min_p * p.max()
    q = torch.where(keep, p, torch.zeros_like(p))
    return q / q.sum()


def inverse_cdf_pick(dist: torch.Tensor, u: float) -> int:
    """First index (in vocabulary order) whose cumulative probability exceeds u."""
    c = torch.cumsum(dist.to(torch.float64), 0)
    idx = int((c <= u).sum().item())
    nz = torch.nonzero(dist > 0).flatten()
    return min(max(idx, int(nz[0])), int(nz[-1]))
