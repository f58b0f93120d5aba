"""Hands out and takes back numbered resources (sequence slots, cache pages).

Host-side bookkeeping only.  An id is either free or held, never both; giving back an id
that is not held, or asking for more than there is, raises instead of corrupting the pool.
"""
from __future__ import annotations

import heapq


class CacheFull(RuntimeError):
    """The cache has no room for what a step needs (pages or sequence slots)."""


class CacheError(RuntimeError):
    """Misuse of the cache: unknown or already freed slot or page."""


class IdPool:
    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n))   # a heap: the lowest id is reused first
        self._held: set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = heapq.heappop(self._free)
        self._held.add(i)
        return i

    def alloc_many(self, k: int) -> list[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.alloc() for _ in range(k)]

    def free(self, i: int) -> None:
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is not held (freed twice, or never given out)")
        self._held.remove(i)
        heapq.heappush(self._free, i)

    def holds(self, i: int) -> bool:
        return i in self._held

    def check(self) -> None:
        """Every id is exactly once in free or held."""
        free = sorted(self._free)
        assert len(set(free)) == len(free), f"{self.what}: an id is free twice"
        assert not (set(free) & self._held), f"{self.what}: an id is free and held"
        assert len(free) + len(self._held) == self.n, f"{self.what}: an id was lost"
