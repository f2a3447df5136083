"""Dispatch of paged attention to the kernel that takes the shape.

The general kernel (one warp per token and head) takes every supported shape in both
storage types; tuned kernels register themselves for the shapes they cover. A shape no
kernel takes raises, it never computes something else.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def paged_attention(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    page_stride: int, ctx, group, nq: int, nkv: int, hd: int, scale: float,
                    window: Optional[int]) -> torch.Tensor:
    """q [tokens, nq*hd] (row stride free) -> out [tokens, nq*hd], over the pages that
    ``group.block_table`` lists for each request of the step."""
    for impl in _TUNED:
        if impl(q, out, k_cache, v_cache, page_stride, ctx, group, nq, nkv, hd, scale, window):
            return out
    return ops.attention_generic(q, out, k_cache, v_cache, page_stride, ctx.cache.page_size,
                                 group.block_table, ctx.token_req, ctx.positions, nq, nkv, hd, scale, window)


# tuned implementations: fn(...) -> bool, True when it ran
_TUNED = []


def register_tuned(fn) -> None:
    _TUNED.append(fn)


# ---------------------------------------------------------------------------
# tensor-core kernel (bfloat16, head_dim 32 / 64 / 128): host-side planning of work items
# ---------------------------------------------------------------------------
import dataclasses  # noqa: E402
from ctypes import c_float, c_int, c_longlong, c_void_p  # noqa: E402

import numpy as np  # noqa: E402

from . import lib as _lib  # noqa: E402

_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float
_lib.declare("oi_attention_mma", [_P, _I, _P, _I, _P, _P, _L, _I, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I,
                                  _F, _I, _P, _P, _I, _P])

ROWS_PER_CTA = 64
KEYS_PER_TILE = 64
MAX_SPLITS = 16
MIN_TILES_PER_SPLIT = 2   # a slice of the keys is at least 128 keys long
_SM_COUNT = None


def _sm_count(device) -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT


@dataclasses.dataclass
class AttentionPlan:
    items: torch.Tensor          # int32 [n, 4]: request, first token of the tile, split, nsplits
    row_splits: torch.Tensor     # int32 [tokens]
    num_items: int
    any_split: bool
    max_splits: int
    part_o: Optional[torch.Tensor]
    part_lse: Optional[torch.Tensor]


def plan_items(q_lens, kv_lens, group: int, nkv: int, window: Optional[int], sm_count: int):
    """Work items of one step: for every request its query tiles (64 rows = 64 // group tokens
    times `group` heads); when the grid would leave SMs idle (decode at small batch), a tile's
    keys are cut into slices. Returns (items [n, 4], row_splits [tokens], max_splits)."""
    tpt = ROWS_PER_CTA // group
    tiles = []
    for b, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        for t0 in range(0, n, tpt):
            toks = min(tpt, n - t0)
            pos0 = kv - n + t0
            lo = (max(0, pos0 - window + 1) if window else 0) & ~(KEYS_PER_TILE - 1)
            span_tiles = -(-(pos0 + toks - lo) // KEYS_PER_TILE)
            tiles.append((b, t0, toks, span_tiles))
    want = 1
    if len(tiles) * nkv < 2 * sm_count:
        want = min(MAX_SPLITS, -(-2 * sm_count // (len(tiles) * nkv)))
    items = []
    row_splits = np.ones(sum(q_lens), dtype=np.int32)
    starts = np.concatenate([[0], np.cumsum(q_lens)])
    max_splits = 1
    for b, t0, toks, span_tiles in tiles:
        ns = max(1, min(want, span_tiles // MIN_TILES_PER_SPLIT))
        max_splits = max(max_splits, ns)
        row_splits[starts[b] + t0: starts[b] + t0 + toks] = ns
        for s in range(ns):
            items.append((b, t0, s, ns))
    return np.asarray(items, dtype=np.int32).reshape(-1, 4), row_splits, max_splits


def plan_items_static_decode(num_requests: int, nkv: int, sm_count: int):
    """Items of a decode step whose launch is recorded once and replayed (a CUDA graph): one
    query token per request, and a number of key slices that depends on the batch size only;
    the kernel finds each slice's bounds from the request's current length."""
    ns = 1
    if num_requests * nkv < 2 * sm_count:
        ns = min(MAX_SPLITS, -(-2 * sm_count // (num_requests * nkv)))
    items = np.asarray([(b, 0, s, ns) for b in range(num_requests) for s in range(ns)], dtype=np.int32)
    return items.reshape(-1, 4), np.full(num_requests, ns, dtype=np.int32), ns


def _plan_for(ctx, group_step, group: int, nq: int, nkv: int, hd: int, window, device) -> AttentionPlan:
    key = ("attention_mma_plan", id(group_step), group, nkv, window)
    plan = ctx.scratch.get(key)
    if plan is None:
        if getattr(ctx, "static_decode", False):
            items, row_splits, max_splits = plan_items_static_decode(ctx.num_requests, nkv, _sm_count(device))
        else:
            items, row_splits, max_splits = plan_items(ctx.q_lens_host, ctx.kv_lens_host, group, nkv, window,
                                                       _sm_count(device))
        any_split = max_splits > 1
        packed = np.concatenate([items.reshape(-1), row_splits])
        dev = torch.from_numpy(packed).to(device, non_blocking=True)
        n = items.shape[0]
        part_o = part_lse = None
        if any_split:
            part_o = torch.empty(ctx.num_tokens * nq * max_splits * hd, dtype=torch.float32, device=device)
            part_lse = torch.empty(ctx.num_tokens * nq * max_splits, dtype=torch.float32, device=device)
        plan = AttentionPlan(dev[: n * 4].view(n, 4), dev[n * 4:], n, any_split, max_splits, part_o, part_lse)
        ctx.scratch[key] = plan
    return plan


def attention_mma(q, out, k_cache, v_cache, page_stride, ctx, group_step, nq, nkv, hd, scale, window) -> bool:
    """The tensor-core kernel, when it covers the shape: bfloat16, head_dim 32, 64 or 128."""
    if q.dtype != torch.bfloat16 or hd not in (32, 64, 128) or nq // nkv > ROWS_PER_CTA:
        return False
    if q.stride(0) % 2 or page_stride % 8:
        return False
    plan = getattr(ctx, "attention_plan_override", None) or _plan_for(
        ctx, group_step, nq // nkv, nq, nkv, hd, window, q.device)
    L = _lib.load()
    _lib.check(L.oi_attention_mma(
        q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
        int(page_stride), ctx.cache.page_size, group_step.block_table.data_ptr(), group_step.block_table.stride(0),
        ctx.cu_seqlens.data_ptr(), group_step.kv_lens.data_ptr(), plan.items.data_ptr(), plan.num_items,
        plan.row_splits.data_ptr(), out.shape[0], 1 if plan.any_split else 0, nq, nkv, hd, float(scale),
        int(window) if window else 0, 0 if plan.part_o is None else plan.part_o.data_ptr(),
        0 if plan.part_lse is None else plan.part_lse.data_ptr(), plan.max_splits,
        torch.cuda.current_stream().cuda_stream), "attention_mma")
    return True


register_tuned(attention_mma)
