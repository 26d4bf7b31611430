"""Index allocators for sequence slots and cache pages.

The reference ties a sequence to its batch row for the life of a plan
(engine/model.py:229-235); here a slot is taken when a sequence starts,
given back when its batch ends, and used again by a later batch.
"""

from __future__ import annotations

import heapq
from typing import List


class CacheError(RuntimeError):
    """The cache cannot serve a request (no slot or page left, bad slot, capacity exceeded)."""


class IndexAllocator:
    """Hands out the integers 0..n-1, lowest free first; every index is either free or held, never both."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n))
        heapq.heapify(self._free)
        self._held = set()

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.n} are in use")
        i = heapq.heappop(self._free)
        self._held.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never taken)")
        self._held.remove(i)
        heapq.heappush(self._free, i)

    def holds(self, i: int) -> bool:
        return i in self._held

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def check(self) -> None:
        """Every index is accounted for exactly once."""
        free = sorted(self._free)
        if len(set(free)) != len(free) or set(free) & self._held or len(free) + len(self._held) != self.n:
            raise CacheError(f"{self.what} allocator is inconsistent: {len(free)} free, {len(self._held)} held of {self.n}")
