"""The cache manager: paged keys and values with a block table per request, in groups of
layers that share a geometry, and slots for per-request state of fixed size.

A *group* is the set of layers (more exactly: of calls in the model's run order)
whose mixers asked for the same (kv heads, head size, window). Each group has a
pool of pages of its own; a page id names ``page_size`` positions of every layer of
the group, K and V. The device tensor is laid out layer first,
``[layers_in_group, 2, pages, page_size, kv_heads, head_dim]``: what one layer's
attention reads in a step then lies in two dense regions (its K pages and its V pages)
instead of being strewn over the whole pool at a stride of one page of all layers, as in
the reference's page-first buffer (pegainfer-kv-cache/src/layout.rs:5-33), which keeps
the address translation and the DRAM rows of a layer's pass local. A request holds, per group, a block table:
page ids in position order. Pages go back to the pool when the request ends, or,
in a group with a window, as soon as every position of the page is further back
than the window of any query still to come.

The two-phase protocol follows the reference's ``schedule_* / apply_*``
(kvbm/kvbm-logical/src/integrations/scheduled.rs:469-661): ``reserve`` takes the
pages a step needs and changes nothing when they are not there; ``commit`` advances
the request after the step ran; ``rollback`` undoes a reservation.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .pool import IdPool, OutOfPages

RELEASED = -1  # block-table entry of a page that a window has left behind


@dataclasses.dataclass(frozen=True)
class KvNeed:
    """What an attention-like mixer asks of the cache."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # keys a query sees, itself included; None = all


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (a recurrent or convolution state)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"  # "float32" or "model" (the model's activation dtype)


@dataclasses.dataclass(frozen=True)
class KvHandle:
    group: int
    layer: int  # index inside the group


@dataclasses.dataclass
class _Group:
    need: KvNeed
    layers: int = 0
    pool: Optional[IdPool] = None
    tensor: object = None  # torch.Tensor once allocated

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclasses.dataclass
class _Request:
    tables: List[List[int]]          # per group: page id per page index, RELEASED where freed
    num_tokens: int = 0              # positions whose keys are in the cache
    reserved: int = 0                # tokens reserved beyond num_tokens by the step in flight
    new_pages: Optional[List[List[int]]] = None  # pages taken by that reservation, per group
    state_slot: int = -1


class CacheManager:
    def __init__(self, page_size: int = 16) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.groups: List[_Group] = []
        self.state_needs: List[StateNeed] = []
        self.state_tensors: List[object] = []
        self.slot_pool: Optional[IdPool] = None
        self.requests: Dict[Hashable, _Request] = {}
        self._allocated = False

    # ------------------------------------------------------------------
    # set-up: mixers register their needs, then memory is allocated once
    # ------------------------------------------------------------------
    def add_kv_layer(self, need: KvNeed) -> KvHandle:
        if self._allocated:
            raise RuntimeError("cache needs must be registered before allocation")
        if need.window is not None and need.window <= 0:
            raise ValueError(f"window must be positive, got {need.window}")
        for gi, g in enumerate(self.groups):
            if g.need == need:
                g.layers += 1
                return KvHandle(gi, g.layers - 1)
        self.groups.append(_Group(need=need, layers=1))
        return KvHandle(len(self.groups) - 1, 0)

    def add_state(self, need: StateNeed) -> int:
        if self._allocated:
            raise RuntimeError("cache needs must be registered before allocation")
        self.state_needs.append(need)
        return len(self.state_needs) - 1

    def bytes_per_page(self, group: int, element_size: int) -> int:
        g = self.groups[group]
        return g.layers * 2 * self.page_size * g.need.num_kv_heads * g.need.head_dim * element_size

    def bytes_per_token(self, element_size: int) -> int:
        """Cache bytes one position costs over all groups (windows not counted as savings)."""
        return sum(self.bytes_per_page(i, element_size) for i in range(len(self.groups))) // self.page_size

    def allocate(self, num_pages: int, max_requests: int, device=None, dtype=None) -> None:
        """Create the pools (and, when ``device`` is given, the device tensors).

        Every group gets ``num_pages`` pages. ``max_requests`` is the number of state
        slots, i.e. of requests that may be open at once.
        """
        if self._allocated:
            raise RuntimeError("already allocated")
        if num_pages <= 0 or max_requests <= 0:
            raise ValueError("num_pages and max_requests must be positive")
        self.num_pages = num_pages
        self.max_requests = max_requests
        for g in self.groups:
            g.pool = IdPool(num_pages, "page")
        self.slot_pool = IdPool(max_requests, "state slot")
        if device is not None:
            import torch

            for g in self.groups:
                g.tensor = torch.zeros(
                    (g.layers, 2, num_pages, self.page_size, g.need.num_kv_heads, g.need.head_dim),
                    dtype=dtype, device=device)
            for need in self.state_needs:
                sdtype = dtype if need.dtype == "model" else torch.float32
                self.state_tensors.append(torch.zeros((max_requests, *need.shape), dtype=sdtype, device=device))
        self._allocated = True

    # ------------------------------------------------------------------
    # device views for the mixers
    # ------------------------------------------------------------------
    def kv_views(self, handle: KvHandle):
        """(k, v, page_stride in elements) of one layer: k and v are views
        [pages, page_size, kv_heads, head_dim] into the group's tensor."""
        t = self.groups[handle.group].tensor
        if t is None:
            raise RuntimeError("the cache has no device memory (allocate(device=...) first)")
        return t[handle.layer, 0], t[handle.layer, 1], t.stride(2)

    def state_tensor(self, state_id: int):
        return self.state_tensors[state_id]

    # ------------------------------------------------------------------
    # page arithmetic
    # ------------------------------------------------------------------
    def pages_for(self, tokens: int) -> int:
        return -(-tokens // self.page_size)

    def _first_needed_page(self, g: _Group, start: int) -> int:
        """Lowest page index a query at position >= start can read in group g."""
        if g.window is None:
            return 0
        first_key = max(0, start - g.window + 1)
        return first_key // self.page_size

    def pages_needed(self, request_id: Hashable, new_tokens: int) -> List[int]:
        """Pages per group a reservation of ``new_tokens`` more positions would take."""
        r = self.requests[request_id]
        end = r.num_tokens + r.reserved + new_tokens
        return [max(0, self.pages_for(end) - len(r.tables[gi])) for gi in range(len(self.groups))]

    def free_pages(self) -> List[int]:
        return [g.pool.free_count for g in self.groups]

    def min_free_pages(self) -> int:
        return min((g.pool.free_count for g in self.groups), default=self.num_pages)

    # ------------------------------------------------------------------
    # request life cycle
    # ------------------------------------------------------------------
    def open(self, request_id: Hashable) -> int:
        """Start a request: an empty block table per group and a state slot. Returns the slot."""
        if request_id in self.requests:
            raise KeyError(f"request {request_id!r} is already open")
        slot = self.slot_pool.allocate(1)[0]  # raises OutOfPages when all slots are taken
        for t in self.state_tensors:
            t[slot].zero_()
        self.requests[request_id] = _Request(tables=[[] for _ in self.groups], state_slot=slot)
        return slot

    def has(self, request_id: Hashable) -> bool:
        return request_id in self.requests

    def num_tokens(self, request_id: Hashable) -> int:
        return self.requests[request_id].num_tokens

    def state_slot(self, request_id: Hashable) -> int:
        return self.requests[request_id].state_slot

    def reserve(self, request_id: Hashable, new_tokens: int) -> int:
        """Take the pages for positions [n, n + new_tokens) in every group; returns n.

        Raises OutOfPages and changes nothing if any group cannot supply them."""
        r = self.requests[request_id]
        if r.reserved:
            raise RuntimeError(f"request {request_id!r} already has a reservation in flight")
        if new_tokens <= 0:
            raise ValueError("new_tokens must be positive")
        need = self.pages_needed(request_id, new_tokens)
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.free_count:
                raise OutOfPages(
                    f"request {request_id!r}: group {gi} needs {need[gi]} pages, {g.pool.free_count} free")
        taken: List[List[int]] = []
        for gi, g in enumerate(self.groups):
            pages = g.pool.allocate(need[gi])
            r.tables[gi].extend(pages)
            taken.append(pages)
        r.reserved = new_tokens
        r.new_pages = taken
        return r.num_tokens

    def rollback(self, request_id: Hashable) -> None:
        """Give back what the reservation in flight took (the step did not run)."""
        r = self.requests[request_id]
        if not r.reserved:
            return
        for gi, g in enumerate(self.groups):
            pages = r.new_pages[gi]
            if pages:
                del r.tables[gi][len(r.tables[gi]) - len(pages):]
                g.pool.release(pages)
        r.reserved = 0
        r.new_pages = None

    def commit(self, request_id: Hashable) -> None:
        """The reserved positions are now in the cache. Pages that every later query's
        window has passed go back to their pool."""
        r = self.requests[request_id]
        if not r.reserved:
            raise RuntimeError(f"request {request_id!r} has no reservation to commit")
        r.num_tokens += r.reserved
        r.reserved = 0
        r.new_pages = None
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            first = self._first_needed_page(g, r.num_tokens)
            table = r.tables[gi]
            dead = [p for p in table[:first] if p != RELEASED]
            if dead:
                g.pool.release(dead)
                for i in range(min(first, len(table))):
                    table[i] = RELEASED

    def close(self, request_id: Hashable) -> None:
        """End a request: all its pages and its state slot go back."""
        r = self.requests.pop(request_id)
        for gi, g in enumerate(self.groups):
            g.pool.release([p for p in r.tables[gi] if p != RELEASED])
        self.slot_pool.release([r.state_slot])

    def block_table(self, request_id: Hashable, group: int) -> Sequence[int]:
        return self.requests[request_id].tables[group]

    # ------------------------------------------------------------------
    def check(self) -> None:
        """Invariants over pools and tables: no page lost, none held twice."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = set()
            for rid, r in self.requests.items():
                for p in r.tables[gi]:
                    if p == RELEASED:
                        continue
                    if p in seen:
                        raise AssertionError(f"page {p} of group {gi} is in two tables")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"page {p} of group {gi} is in a table but free")
                    seen.add(p)
            if len(seen) != g.pool.used_count:
                raise AssertionError(
                    f"group {gi}: {g.pool.used_count} pages held but {len(seen)} in tables")
        self.slot_pool.check()
        slots = [r.state_slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slot_pool.used_count:
            raise AssertionError("state slots and open requests disagree")
