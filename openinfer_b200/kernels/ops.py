"""Python wrappers of the CUDA entry points: shape and dtype checks, pointers, error mapping.

Every function takes torch tensors that live on the CUDA device and launches on
the current stream. None of them has another implementation to fall back to.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError

_DT = {torch.float32: 0, torch.bfloat16: 1}


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError(
                "a kernel was given a tensor that is not on a CUDA device; "
                "this package has no CPU path"
            )


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return _lib.current_stream()


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous()):
        raise KernelError(f"{what} must be a contiguous int32 tensor")


def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :]"""
    _cuda(out, table, ids)
    _i32(ids, "embedding ids")
    tokens, hidden = out.shape
    if table.shape[1] != hidden or ids.numel() != tokens or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError(f"embedding: shapes out={tuple(out.shape)} table={tuple(table.shape)} ids={tuple(ids.shape)}")
    L = _lib.load()
    _lib.check(L.oi_embedding(out.data_ptr(), _code(out, "embedding"), table.data_ptr(), _code(table, "embedding"),
                              ids.data_ptr(), tokens, hidden, table.shape[0], _stream()), "embedding")
    return out


def gather_tokens(ids: torch.Tensor, src: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """ids[i] = tokens[src[i]] wherever src[i] >= 0 (all int32, on the device)."""
    _cuda(ids, src, tokens)
    _i32(ids, "gather_tokens ids")
    _i32(src, "gather_tokens src")
    _i32(tokens, "gather_tokens tokens")
    if ids.numel() != src.numel() or not (ids.is_contiguous() and src.is_contiguous() and tokens.is_contiguous()):
        raise KernelError("gather_tokens: ids and src must be contiguous and of one length")
    L = _lib.load()
    _lib.check(L.oi_gather_tokens(ids.data_ptr(), src.data_ptr(), tokens.data_ptr(), ids.numel(), tokens.numel(),
                                  _stream()), "gather_tokens")
    return ids


def copy_words(dst: torch.Tensor, src: torch.Tensor, n: int, *, ids_off: int = -1, src_off: int = 0, n_ids: int = 0,
               tokens: Optional[torch.Tensor] = None, fence: bool = False) -> None:
    """dst[:n] = src[:n] (int32) by a kernel; one of the two may be pinned host memory, which the device
    reads or writes directly. With ``ids_off >= 0`` the words [ids_off, ids_off + n_ids) are token ids:
    where the source index at ``src_off`` is >= 0 the id comes from ``tokens`` (int32, on the device).
    ``fence``: what is copied is read by later kernels before their own wait for their predecessor (a step's
    lengths, block tables, positions, work items): the kernel launched next then gets plain stream order."""
    for t, what in ((dst, "dst"), (src, "src")):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.numel() < n or not (t.is_cuda or t.is_pinned()):
            raise KernelError(f"copy_words: {what} must be contiguous int32 of at least {n} words, on the device or pinned")
    if tokens is not None:
        _cuda(tokens)
        _i32(tokens, "copy_words tokens")
    L = _lib.load()
    _lib.check(L.oi_copy_words(dst.data_ptr(), src.data_ptr(), int(n), int(ids_off), int(src_off), int(n_ids),
                               _ptr(tokens), 0 if tokens is None else tokens.numel(), _stream()), "copy_words")
    if fence:
        L.oi_launch_fence()


class UploadRing:
    """Small host arrays of int32 to the device without a copy-engine operation and without making the host wait
    for the stream: a ring of pinned buffers that a kernel reads (``copy_words``), each guarded by the event of its
    last use."""

    def __init__(self, slots: int = 4) -> None:
        self.slots = slots
        self.buffers: list = []
        self.events: list = []
        self.turn = 0

    def upload(self, host, device) -> torch.Tensor:
        n = int(host.size)
        if not self.buffers or self.buffers[0].numel() < n:
            if self.buffers:
                torch.cuda.current_stream().synchronize()   # kernels in flight may still read the old buffers
            self.buffers = [torch.empty(max(4096, 2 * n), dtype=torch.int32, pin_memory=True) for _ in range(self.slots)]
            self.events = [None] * self.slots
        self.turn = (self.turn + 1) % self.slots
        if self.events[self.turn] is not None:
            self.events[self.turn].synchronize()
        buf = self.buffers[self.turn]
        buf[:n].numpy()[:] = host
        dev = torch.empty(max(n, 1), dtype=torch.int32, device=device)
        if n:
            copy_words(dev, buf, n, fence=True)
        event = torch.cuda.Event()
        event.record()
        self.events[self.turn] = event
        return dev[:n]


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float, *,
            delta: Optional[torch.Tensor] = None, row_idx: Optional[torch.Tensor] = None,
            weight_offset: float = 0.0) -> torch.Tensor:
    """out = x * rsqrt(mean(x^2) + eps) * (weight_offset + weight), row by row.

    ``delta``: x <- x + delta first (stored in x), the norm is of the sum.
    ``row_idx``: output row r reads x[row_idx[r]].
    """
    _cuda(out, x, weight, delta, row_idx)
    _i32(row_idx, "rmsnorm row_idx")
    hidden = x.shape[-1]
    rows = out.shape[0]
    if out.dtype != x.dtype or (delta is not None and (delta.dtype != x.dtype or delta.shape != x.shape)):
        raise KernelError("rmsnorm: out, x and delta must share a dtype and shape")
    if not (out.is_contiguous() and x.is_contiguous() and weight.is_contiguous()) or weight.numel() != hidden:
        raise KernelError(f"rmsnorm: shapes x={tuple(x.shape)} weight={tuple(weight.shape)}")
    if delta is not None and not delta.is_contiguous():
        raise KernelError("rmsnorm: delta must be contiguous")
    if out.shape[-1] != hidden or (row_idx is None and rows != x.shape[0]) or (row_idx is not None and row_idx.numel() != rows):
        raise KernelError("rmsnorm: row counts do not match")
    L = _lib.load()
    _lib.check(L.oi_rmsnorm(out.data_ptr(), x.data_ptr(), _ptr(delta), _code(x, "rmsnorm"), weight.data_ptr(),
                            _code(weight, "rmsnorm weight"), _ptr(row_idx), rows, hidden, float(eps),
                            float(weight_offset), _stream()), "rmsnorm")
    return out


def add_inplace(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _cuda(x, delta)
    if x.dtype != delta.dtype or x.shape != delta.shape or not (x.is_contiguous() and delta.is_contiguous()):
        raise KernelError("add: operands must share dtype and shape and be contiguous")
    L = _lib.load()
    _lib.check(L.oi_add_inplace(x.data_ptr(), delta.data_ptr(), _code(x, "add"), x.numel(), _stream()), "add")
    return x


def scale_cap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place: x = x * scale, then, with cap > 0, x = cap * tanh(x / cap)."""
    _cuda(x)
    if not x.is_contiguous():
        raise KernelError("scale_cap: the tensor must be contiguous")
    L = _lib.load()
    _lib.check(L.oi_scale_cap(x.data_ptr(), _code(x, "scale_cap"), x.numel(), float(scale), float(cap), _stream()), "scale_cap")
    return x


# gate activations of a gated feed-forward: name -> code of the C interface (common.cuh)
ACTIVATIONS = {"silu": 1, "gelu_tanh": 2}


def act_code(name: str) -> int:
    try:
        return ACTIVATIONS[name]
    except KeyError:
        raise KernelError(f"activation {name!r} has no kernel (known: {', '.join(sorted(ACTIVATIONS))})") from None


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, block: Optional[int] = None, act: str = "silu") -> torch.Tensor:
    """out[r, i] = act(gate_i) * up_i for a fused gate|up buffer [rows, 2 * inter] laid out in
    blocks of ``block`` gate values followed by their up values (default: all gates, then all ups)."""
    _cuda(out, gate_up)
    rows, inter = out.shape
    block = inter if block is None else int(block)
    if gate_up.shape != (rows, 2 * inter) or out.dtype != gate_up.dtype or not (out.is_contiguous() and gate_up.is_contiguous()):
        raise KernelError(f"silu_mul: shapes out={tuple(out.shape)} gate_up={tuple(gate_up.shape)}")
    L = _lib.load()
    _lib.check(L.oi_silu_mul(out.data_ptr(), gate_up.data_ptr(), _code(out, "silu_mul"), rows, inter, block, act_code(act),
                             _stream()), "silu_mul")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, nq: int, nkv: int, hd: int, *, q_norm_w: Optional[torch.Tensor],
                    k_norm_w: Optional[torch.Tensor], eps: float, weight_offset: float,
                    cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], positions: torch.Tensor,
                    slots: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                    v_cache: Optional[torch.Tensor], page_stride: int, page_size: int,
                    write_kv: bool = True, interleaved: bool = False) -> None:
    """Per-head norm and rotation of q (in place) and k, and the write of k and v into
    their pages. ``qkv`` is [tokens, >= (nq + 2 nkv) * hd] (or [tokens, >= nq * hd] when
    write_kv is false); ``cos``/``sin`` are float32 [max_pos, rotary_dim / 2]; ``interleaved``: angle d turns the
    neighbours (2 d, 2 d + 1) instead of (d, d + rotary_dim / 2)."""
    _cuda(qkv, q_norm_w, k_norm_w, cos, sin, positions, slots, k_cache, v_cache)
    _i32(positions, "positions")
    _i32(slots, "slots")
    tokens = qkv.shape[0]
    width = (nq + 2 * nkv) * hd if write_kv else nq * hd
    if qkv.dim() != 2 or qkv.shape[1] < width or qkv.stride(1) != 1:
        raise KernelError(f"qk_norm_rope_kv: qkv shape {tuple(qkv.shape)} too narrow for {width}")
    if positions.numel() != tokens or (slots is not None and slots.numel() != tokens):
        raise KernelError("qk_norm_rope_kv: positions/slots length differs from the token count")
    norm_code = 0
    for w in (q_norm_w, k_norm_w):
        if w is not None:
            if w.numel() != hd or not w.is_contiguous():
                raise KernelError("qk_norm_rope_kv: norm weight must have head_dim elements")
            norm_code = _code(w, "qk norm weight")
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("qk_norm_rope_kv: q and k norm weights must share a dtype")
    rot_half, max_pos = 0, 0
    if cos is not None:
        if cos.dtype != torch.float32 or sin is None or sin.shape != cos.shape or not (cos.is_contiguous() and sin.is_contiguous()):
            raise KernelError("qk_norm_rope_kv: cos/sin must be contiguous float32 tables of one shape")
        max_pos, rot_half = cos.shape
    if write_kv:
        if k_cache is None or v_cache is None or slots is None or k_cache.dtype != qkv.dtype:
            raise KernelError("qk_norm_rope_kv: the cache must be given and share qkv's dtype")
    L = _lib.load()
    _lib.check(L.oi_qk_norm_rope_kv(
        qkv.data_ptr(), _code(qkv, "qk_norm_rope_kv"), qkv.stride(0), tokens, nq, nkv, hd, _ptr(q_norm_w),
        _ptr(k_norm_w), norm_code, float(eps), float(weight_offset), _ptr(cos), _ptr(sin), rot_half, max_pos,
        positions.data_ptr(), _ptr(slots), _ptr(k_cache), _ptr(v_cache), int(page_stride), int(page_size),
        1 if write_kv else 0, 1 if interleaved else 0, _stream()), "qk_norm_rope_kv")


def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      page_stride: int, page_size: int, block_table: torch.Tensor, token_req: torch.Tensor,
                      positions: torch.Tensor, nq: int, nkv: int, hd: int, scale: float,
                      window: Optional[int] = None) -> torch.Tensor:
    """Paged causal attention, one warp per (token, head). ``q`` is [tokens, >= nq*hd] with
    any row stride; ``out`` is [tokens, nq*hd]; ``block_table`` is int32 [requests, max_pages]."""
    _cuda(q, out, k_cache, v_cache, block_table, token_req, positions)
    _i32(block_table, "block_table")
    _i32(token_req, "token_req")
    _i32(positions, "positions")
    tokens = out.shape[0]
    if q.shape[0] != tokens or q.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != nq * hd:
        raise KernelError(f"attention: shapes q={tuple(q.shape)} out={tuple(out.shape)}")
    if q.dtype != out.dtype or q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise KernelError("attention: q, out and the cache must share a dtype")
    L = _lib.load()
    _lib.check(L.oi_attention_generic(
        q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), _code(q, "attention"), k_cache.data_ptr(),
        v_cache.data_ptr(), int(page_stride), int(page_size), block_table.data_ptr(), block_table.stride(0),
        token_req.data_ptr(), positions.data_ptr(), tokens, nq, nkv, hd, float(scale),
        int(window) if window else 0, _stream()), "attention")
    return out


def gemm_generic(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T, float32 accumulation on the ordinary pipes, k ascending."""
    _cuda(out, a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: shapes a={tuple(a.shape)} w={tuple(w.shape)} out={tuple(out.shape)}")
    L = _lib.load()
    _lib.check(L.oi_gemm_generic(out.data_ptr(), _code(out, "gemm out"), a.data_ptr(), _code(a, "gemm a"),
                                 w.data_ptr(), _code(w, "gemm w"), M, N, K, a.stride(0), w.stride(0),
                                 out.stride(0), _stream()), "gemm")
    return out


def argmax(out: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """out[r] = index of the largest logit of row r (lowest index on ties)."""
    _cuda(out, logits)
    _i32(out, "argmax out")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.numel() != rows:
        raise KernelError("argmax: logits must be float32 rows")
    L = _lib.load()
    nchunks = -(-vocab // 4096)
    pv = pi = None
    if nchunks >= 4:  # a large vocabulary: many blocks per row, partial results in scratch
        pv = torch.empty(rows * nchunks, dtype=torch.float32, device=logits.device)
        pi = torch.empty(rows * nchunks, dtype=torch.int32, device=logits.device)
    _lib.check(L.oi_argmax(out.data_ptr(), logits.data_ptr(), rows, vocab, logits.stride(0), _ptr(pv), _ptr(pi),
                           _stream()), "argmax")
    return out


def token_logprobs(logits: torch.Tensor, rows: torch.Tensor, picked: torch.Tensor, ks: torch.Tensor, k_max: int):
    """For the listed rows of float32 ``logits``: (log-softmax of ``picked[i]``, the ``ks[i]`` largest
    log-probabilities [n, k_max], their ids [n, k_max]; unused places -inf / -1). All index tensors int32
    on the device."""
    _cuda(logits, rows, picked, ks)
    for t, what in ((rows, "rows"), (picked, "picked"), (ks, "ks")):
        _i32(t, f"token_logprobs {what}")
    n = rows.numel()
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or picked.numel() != n or ks.numel() != n:
        raise KernelError("token_logprobs: logits must be float32 rows; rows, picked and ks of one length")
    lp = torch.empty(n, dtype=torch.float32, device=logits.device)
    vals = torch.empty((n, max(k_max, 1)), dtype=torch.float32, device=logits.device)
    ids = torch.empty((n, max(k_max, 1)), dtype=torch.int32, device=logits.device)
    L = _lib.load()
    _lib.check(L.oi_token_logprobs(logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(), picked.data_ptr(),
                                   ks.data_ptr(), n, int(k_max), lp.data_ptr(), vals.data_ptr(), ids.data_ptr(), _stream()),
               "token_logprobs")
    return lp, vals[:, :k_max], ids[:, :k_max]


def sample_use_clusters(on: bool) -> None:
    """Whether rows that can be read 16 bytes at a time are sampled by a cluster of CTAs per row (the default) or
    every row by one block (what the clusters leave unanswered always is)."""
    _lib.check(_lib.load().oi_sample_use_clusters(1 if on else 0), "sample_use_clusters")


def sample(out: torch.Tensor, logits: torch.Tensor, probs_scratch: torch.Tensor, temperature: torch.Tensor,
           top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor, uniform: torch.Tensor) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) after top-k, top-p and min-p,
    by inverse CDF at ``uniform[r]`` in [0, 1)."""
    _cuda(out, logits, probs_scratch, temperature, top_k, top_p, min_p, uniform)
    _i32(out, "sample out")
    _i32(top_k, "top_k")
    rows, vocab = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 rows")
    for t, name in ((temperature, "temperature"), (top_p, "top_p"), (min_p, "min_p"), (uniform, "uniform")):
        if t.dtype != torch.float32 or t.numel() != rows or not t.is_contiguous():
            raise KernelError(f"sample: {name} must be float32 with one entry per row")
    if top_k.numel() != rows or out.numel() != rows:
        raise KernelError("sample: top_k/out must have one entry per row")
    if probs_scratch.dtype != torch.float32 or probs_scratch.numel() < rows * vocab or not probs_scratch.is_contiguous():
        raise KernelError("sample: scratch must hold rows * vocab float32 values")
    L = _lib.load()
    _lib.check(L.oi_sample(out.data_ptr(), logits.data_ptr(), logits.stride(0), probs_scratch.data_ptr(), rows, vocab,
                           temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), min_p.data_ptr(),
                           uniform.data_ptr(), _stream()), "sample")
    return out
