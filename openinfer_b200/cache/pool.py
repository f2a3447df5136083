"""Fixed-size pools: pages of keys and values, and slots of per-request state.

Host-side bookkeeping only; the device memory the ids refer to is owned by
``CacheManager``. The reference keeps the same split between a logical block
pool and one device buffer (pegainfer-kv-cache/src/pool.rs:31-244,
pegainfer-kv-cache/src/buffer.rs:21-71).
"""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """A reservation needs more pages (or slots) than are free. Nothing was taken."""


class DoubleFree(RuntimeError):
    """An id was given back that is not held."""


class IdPool:
    """Ids 0..n-1; each is either free or held by exactly one owner.

    Freed ids are handed out again first (last freed, first reused), so reuse of a
    page shows up in tests as soon as possible. Ids that are given back together come
    out again in ascending order, as a fresh pool's do: pages with consecutive ids lie
    side by side in the cache, and the prompt attention kernel fetches such a run with
    one copy.
    """

    def __init__(self, count: int, what: str = "page") -> None:
        if count < 0:
            raise ValueError(f"{what} count must be >= 0, got {count}")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count - 1, -1, -1))  # pop() gives 0 first
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.count - len(self._free)

    def allocate(self, n: int) -> List[int]:
        """Take n ids, or raise OutOfPages and take none."""
        if n < 0:
            raise ValueError("n must be >= 0")
        if n > len(self._free):
            raise OutOfPages(f"need {n} {self.what}s, {len(self._free)} of {self.count} free")
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._held[i] = True
        return out

    def release(self, ids: Iterable[int]) -> None:
        ids = list(ids)
        seen = set()
        for i in ids:  # all or nothing: check everything before anything changes
            if not (0 <= i < self.count) or not self._held[i] or i in seen:
                raise DoubleFree(f"{self.what} {i} is not held")
            seen.add(i)
        for i in sorted(ids, reverse=True):   # pop() takes from the end: the smallest of these first
            self._held[i] = False
            self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]

    def check(self) -> None:
        """Invariants: every id is in exactly one of free / held."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"{self.what} listed free twice")
        for i in range(self.count):
            if self._held[i] == (i in free):
                raise AssertionError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")
