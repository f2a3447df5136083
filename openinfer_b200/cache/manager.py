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

Prefix cache (optional; the reference's is on by default, kvbm-logical scheduled.rs:436-459): a FULL
page of PROMPT tokens is registered under a lineage key, the digest of (its parent's key, its token ids).
A new request's prompt is matched page by page from the front; matched pages are shared (counted
references, never written again: only positions behind them are), and at least one prompt token is
always left to compute. When the last reference goes the page stays registered but idle, and idle pages
are evicted, least recently used first and leaves before their parents, when a reservation needs room.
It is only used when no group has a window and no mixer keeps state of its own (neither can be restored
from pages).

The two-phase protocol follows the reference's ``schedule_* / apply_*``
(kvbm/kvbm-logical/src/integrations/scheduled.rs:469-661): ``reserve`` takes the
pages a step needs and changes nothing when they are not there; ``commit`` advances
the request after the step ran; ``rollback`` undoes a reservation.
"""
from __future__ import annotations

import collections
import dataclasses
import hashlib
import struct
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
class _Block:
    """A registered full page of prompt tokens: one page id per group, and who uses it."""

    key: bytes
    pages: List[int]
    refs: int = 0


@dataclasses.dataclass
class _Request:
    tables: List[List[int]]          # per group: page id per page index, RELEASED where freed
    num_tokens: int = 0              # positions whose keys are in the cache
    reserved: int = 0                # tokens reserved beyond num_tokens by the step in flight
    new_pages: Optional[List[List[int]]] = None  # pages taken by that reservation, per group
    state_slot: int = -1
    # prefix cache: the registered blocks behind table entries [0, len(blocks)); the lineage key after
    # them; tokens known beyond them; whether further pages may still be registered
    blocks: List[_Block] = dataclasses.field(default_factory=list)
    chain: bytes = b""
    known: List[int] = dataclasses.field(default_factory=list)
    registering: bool = False


def _lineage(parent: bytes, tokens: Sequence[int]) -> bytes:
    return hashlib.blake2b(parent + struct.pack(f"<{len(tokens)}i", *tokens), digest_size=16).digest()


class CacheManager:
    def __init__(self, page_size: int = 16, prefix_cache: bool = False) -> None:
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, got {page_size}")
        self.page_size = page_size
        self.prefix_cache = bool(prefix_cache)
        self._blocks: Dict[bytes, _Block] = {}
        self._idle: "collections.OrderedDict[bytes, _Block]" = collections.OrderedDict()   # no references; oldest first
        self.prefix_hits = 0          # prompt tokens served from registered pages so far
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
        """Pages a reservation could get, per group: free ones and registered ones that nobody uses."""
        return [g.pool.free_count + len(self._idle) for g in self.groups]

    def min_free_pages(self) -> int:
        return min((g.pool.free_count + len(self._idle) for g in self.groups), default=self.num_pages)

    # ------------------------------------------------------------------
    # prefix cache
    # ------------------------------------------------------------------
    def prefix_usable(self) -> bool:
        return self.prefix_cache and not self.state_needs and all(g.window is None for g in self.groups)

    def _evict_for(self, need: Sequence[int]) -> None:
        """Evict idle registered pages until every group can supply ``need`` (checked by the caller to be possible)."""
        while self._idle and any(need[gi] > g.pool.free_count for gi, g in enumerate(self.groups)):
            key, blk = self._idle.popitem(last=False)
            del self._blocks[key]
            for gi, g in enumerate(self.groups):
                g.pool.release([blk.pages[gi]])

    def begin(self, request_id: Hashable, prompt_tokens: Sequence[int]) -> int:
        """Open a request and give it the registered pages that match the front of its prompt.
        Returns how many prompt tokens that covers (a multiple of the page size, and less than the
        prompt: at least one token is left to compute, from which the first logits come)."""
        self.open(request_id)
        if not self.prefix_usable():
            return 0
        r = self.requests[request_id]
        P = self.page_size
        r.registering = True
        for i in range((len(prompt_tokens) - 1) // P):
            key = _lineage(r.chain, prompt_tokens[i * P: (i + 1) * P])
            blk = self._blocks.get(key)
            if blk is None:
                break
            if blk.refs == 0:
                del self._idle[key]
            blk.refs += 1
            r.blocks.append(blk)
            for gi in range(len(self.groups)):
                r.tables[gi].append(blk.pages[gi])
            r.chain = key
        r.num_tokens = len(r.blocks) * P
        self.prefix_hits += r.num_tokens
        return r.num_tokens

    def _register(self, r: _Request, tokens: Optional[Sequence[int]], count: int) -> None:
        """After ``count`` positions were committed: register the pages that they filled, while the token
        ids are known to the host (prompt portions are; tokens still on the device are not)."""
        if not r.registering:
            return
        if tokens is None or len(tokens) != count:
            r.registering = False
            r.known = []
            return
        r.known.extend(int(t) for t in tokens)
        P = self.page_size
        while len(r.known) >= P:
            key = _lineage(r.chain, r.known[:P])
            if key in self._blocks:      # someone else registered the same content meanwhile: ours stays private
                r.registering = False
                r.known = []
                return
            idx = len(r.blocks)
            blk = _Block(key, [r.tables[gi][idx] for gi in range(len(self.groups))], refs=1)
            self._blocks[key] = blk
            r.blocks.append(blk)
            r.chain = key
            del r.known[:P]

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
            if need[gi] > g.pool.free_count + len(self._idle):
                raise OutOfPages(
                    f"request {request_id!r}: group {gi} needs {need[gi]} pages, {g.pool.free_count + len(self._idle)} free")
        self._evict_for(need)
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

    def commit(self, request_id: Hashable, tokens: Optional[Sequence[int]] = None) -> None:
        """The reserved positions are now in the cache. Pages that every later query's
        window has passed go back to their pool. ``tokens``: the ids of those positions when the host
        knows them (the prefix cache registers full pages of them)."""
        r = self.requests[request_id]
        if not r.reserved:
            raise RuntimeError(f"request {request_id!r} has no reservation to commit")
        count = r.reserved
        r.num_tokens += r.reserved
        r.reserved = 0
        r.new_pages = None
        self._register(r, tokens, count)
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
        shared = len(r.blocks)
        for blk in reversed(r.blocks):      # leaves become idle first: they are evicted before their parents
            blk.refs -= 1
            if blk.refs == 0:
                self._idle[blk.key] = blk
        for gi, g in enumerate(self.groups):
            g.pool.release([p for p in r.tables[gi][shared:] if p != RELEASED])
        self.slot_pool.release([r.state_slot])

    def block_table(self, request_id: Hashable, group: int) -> Sequence[int]:
        return self.requests[request_id].tables[group]

    # ------------------------------------------------------------------
    def check(self) -> None:
        """Invariants over pools and tables: no page lost, none held twice."""
        for blk in self._blocks.values():
            users = sum(1 for r in self.requests.values() if blk in r.blocks)
            if users != blk.refs:
                raise AssertionError(f"a registered page counts {blk.refs} users but {users} requests hold it")
            if (blk.refs == 0) != (blk.key in self._idle):
                raise AssertionError("a registered page is idle and in use at once, or neither")
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = set()
            for blk in self._blocks.values():
                p = blk.pages[gi]
                if p in seen or not g.pool.is_held(p):
                    raise AssertionError(f"registered page {p} of group {gi} is listed twice or free")
                seen.add(p)
            for rid, r in self.requests.items():
                for i, p in enumerate(r.tables[gi]):
                    if p == RELEASED:
                        continue
                    if i < len(r.blocks):
                        if r.blocks[i].pages[gi] != p:
                            raise AssertionError(f"request {rid!r}: table entry {i} is not its registered page")
                        continue
                    if p in seen:
                        raise AssertionError(f"page {p} of group {gi} is in two tables")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"page {p} of group {gi} is in a table but free")
                    seen.add(p)
            if len(seen) != g.pool.used_count:
                raise AssertionError(
                    f"group {gi}: {g.pool.used_count} pages held but {len(seen)} in tables or registered")
        self.slot_pool.check()
        slots = [r.state_slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.slot_pool.used_count:
            raise AssertionError("state slots and open requests disagree")
