"""Hand-out and return of numbered resources (sequence slots, cache pages).

Pure host bookkeeping. An index is either free or held by exactly one owner; asking
for more than there are, or returning what is not held, raises.
"""
from __future__ import annotations


class CacheFull(RuntimeError):
    """No free slot or page is left."""


class CacheMisuse(RuntimeError):
    """An index was returned that is not held, or is out of range."""


class IndexPool:
    """``n`` indices; the most recently returned one is handed out first."""

    def __init__(self, n: int, what: str = "index"):
        if n < 0:
            raise ValueError(f"a pool cannot hold {n} entries")
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n - 1, -1, -1))      # pop() yields 0 first
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def held(self) -> list:
        return [i for i, h in enumerate(self._held) if h]

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n} {self.what}s are in use")
        i = self._free.pop()
        self._held[i] = True
        return i

    def acquire_many(self, count: int) -> list:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.acquire() for _ in range(count)]

    def release(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheMisuse(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheMisuse(f"{self.what} {i} is returned but not held")
        self._held[i] = False
        self._free.append(i)

    def check(self) -> None:
        """Every index is free exactly once or held; raises if the books are wrong."""
        if len(set(self._free)) != len(self._free):
            raise CacheMisuse(f"a {self.what} is on the free list twice")
        for i in self._free:
            if self._held[i]:
                raise CacheMisuse(f"{self.what} {i} is both free and held")
        if len(self._free) + sum(self._held) != self.n:
            raise CacheMisuse(f"a {self.what} was lost")
