"""Numbered resources that are handed out and given back: sequence slots and
cache pages.  A resource is never lost, never held twice and never freed
twice; a breach raises instead of corrupting a later batch.
"""
from __future__ import annotations

from typing import List

from ..errors import ContextFull, InvalidArgument


class IndexPool:
    """Indices 0..n-1.  The index given back last is handed out first, so a
    batch that follows another one reuses its slots and pages."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise InvalidArgument(f"a pool of {n} {what}s")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise ContextFull(f"all {self.n} {self.what}s are in use")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not (isinstance(i, int) and 0 <= i < self.n):
            raise InvalidArgument(f"{self.what} {i!r} does not exist (there are {self.n})")
        if not self._held[i]:
            raise InvalidArgument(f"{self.what} {i} is not in use: it cannot be given back")
        self._held[i] = False
        self._free.append(i)

    def check(self) -> None:
        """Every index is either free once or held, never both."""
        free = sorted(self._free)
        assert len(set(free)) == len(free), f"a {self.what} is on the free list twice"
        assert all(not self._held[i] for i in free), f"a free {self.what} is marked held"
        assert len(free) + sum(self._held) == self.n, f"a {self.what} was lost"
