"""A pool of indices (slots or pages) that are taken and given back.

The reference has one sequence and therefore no allocator: its cache only
rewinds a position (crates/mivi-kv/src/cache.rs:287-289).  A batch needs one,
and its three faults are checked here: an index is never lost, never held
twice and never freed twice.
"""
from __future__ import annotations

import heapq
from typing import List


class CacheError(RuntimeError):
    """The cache cannot do what was asked: no slot or page is free, an index is
    given back twice, a sequence would outgrow its capacity."""


class IndexPool:
    def __init__(self, n: int, what: str = "index"):
        if n < 0:
            raise CacheError(f"cannot make a pool of {n} {what}s")
        self.n = n
        self.what = what
        # lowest index first: a freed index is the next one taken, which makes
        # reuse happen early and faults of reuse show in tests.  A heap: a sequence of thousands of
        # pages gives them all back at once when it ends.
        self._free: List[int] = list(range(n))
        self._held = [False] * n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.n} are in use")
        i = heapq.heappop(self._free)
        if self._held[i]:
            raise CacheError(f"{self.what} {i} was on the free list while held")      # cannot happen
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} is outside 0..{self.n - 1}")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held[i] = False
        heapq.heappush(self._free, i)

    def grow(self, n: int) -> None:
        if n < self.n:
            raise CacheError(f"cannot shrink the {self.what} pool from {self.n} to {n}")
        for i in range(self.n, n):
            heapq.heappush(self._free, i)
        self._held += [False] * (n - self.n)
        self.n = n

    def check(self) -> None:
        """Every index is either free once or held, never both."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError(f"a {self.what} is on the free list twice")
        on_list = set(free)
        for i in range(self.n):
            if self._held[i] == (i in on_list):
                raise CacheError(f"{self.what} {i} is {'held and free' if self._held[i] else 'lost'}")
