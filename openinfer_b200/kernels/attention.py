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
