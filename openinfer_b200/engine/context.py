"""What one step looks like to the parts: the flattened batch and its cache metadata.

All rows of a step are one batch: row t belongs to request ``token_req[t]`` at absolute
position ``positions[t]``; request b owns rows ``cu_seqlens[b] .. cu_seqlens[b+1]``
(the reference flattens the same way, pegainfer-qwen3/src/unified_forward.rs:207-223,
pegainfer-kernels/src/ops/attention.rs:396-477). Per cache group there is a slot per row
(page * page_size + offset: where the row's key and value go) and a block table per
request.
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional

import torch


@dataclasses.dataclass
class GroupStep:
    """Cache metadata of one page group for one step (device tensors, int32)."""

    slot_mapping: torch.Tensor   # [tokens]
    block_table: torch.Tensor    # [requests, max_pages]
    kv_lens: torch.Tensor        # [requests] keys visible after this step's rows are written
    window: Optional[int]


@dataclasses.dataclass
class StepContext:
    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor      # int32 [tokens]
    positions: torch.Tensor      # int32 [tokens]
    token_req: torch.Tensor      # int32 [tokens] index of the row's request in this batch
    cu_seqlens: torch.Tensor     # int32 [requests + 1]
    state_slots: torch.Tensor    # int32 [requests] per-request state slot
    groups: List[GroupStep]
    cache: Any                   # CacheManager
    # host copies, for parts that plan launches on the host
    q_lens_host: List[int] = dataclasses.field(default_factory=list)
    starts_host: List[int] = dataclasses.field(default_factory=list)   # position of each request's first row
    kv_lens_host: List[int] = dataclasses.field(default_factory=list)
    state_slots_host: List[int] = dataclasses.field(default_factory=list)
    decode_only: bool = False    # every request brings exactly one row
    max_q_len: int = 0
    max_kv_len: int = 0
    scratch: dict = dataclasses.field(default_factory=dict)  # per-step workspace shared by layers
    # a decode step recorded as a CUDA graph: parts must plan from the batch size alone
    static_decode: bool = False
