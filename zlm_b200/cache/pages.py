"""Host-side bookkeeping of the cache: which pages and which slots are free.
Nothing here touches the GPU; it is plain counting that can be tested anywhere.
"""
from __future__ import annotations

from typing import Iterable, List, Set


class CacheFull(RuntimeError):
    """More tokens or sequences were asked for than the cache was sized for."""


class CacheBookkeepingError(RuntimeError):
    """A page or slot was returned twice, or one that was never handed out."""


class FreeList:
    """Hands out integers 0..n-1, lowest first, and takes them back.  A number is
    never out twice and cannot come back twice."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))     # pop() gives the lowest
        self._held: Set[int] = set()

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self, k: int = 1) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"the cache has {len(self._free)} free {self.what}s, {k} are needed "
                            f"({self.n} in all)")
        out = [self._free.pop() for _ in range(k)]
        self._held.update(out)
        return out

    def give(self, items: Iterable[int]) -> None:
        items = list(items)
        for i in items:
            if i not in self._held:
                raise CacheBookkeepingError(f"{self.what} {i} is returned but is not held")
            self._held.discard(i)
        # keep the free list sorted so that reuse is deterministic (lowest first)
        self._free.extend(items)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every number is either free or held, exactly once."""
        if len(self._free) != len(set(self._free)):
            raise CacheBookkeepingError(f"a {self.what} is on the free list twice")
        if set(self._free) & self._held:
            raise CacheBookkeepingError(f"a {self.what} is both free and held")
        if len(self._free) + len(self._held) != self.n:
            raise CacheBookkeepingError(f"{self.n - len(self._free) - len(self._held)} {self.what}s are lost")
