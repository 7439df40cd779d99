"""Bookkeeping of reusable integer resources (sequence slots, pages of keys).

A ``FreeList`` hands out each number at most once until it is given back, and
refuses a number that is given back twice or was never handed out.  The
reference's cache has no such lifecycle: its batch lives and dies together
(src/detllm/model.py:67-102).
"""

from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """The cache cannot do what was asked (no room, a slot freed twice, ...)."""


class FreeList:
    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * n

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def held(self) -> List[int]:
        return [i for i, h in enumerate(self._held) if h]
