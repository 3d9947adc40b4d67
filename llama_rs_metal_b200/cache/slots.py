"""Host-side bookkeeping of the cache: who holds which slot and which pages.

Pure Python, no device: the tests run it without a GPU. A slot or a page is
either free or held by exactly one owner; taking more than there is, or giving
back what is not held, raises.
"""
from __future__ import annotations

from typing import List

from ..errors import CacheMemoryError, InvalidError


class FreeList:
    """Integers 0..n-1, lowest first out, so that a slot given back is used again at once."""

    def __init__(self, count: int, what: str):
        self.count, self.what = count, what
        self._free = list(range(count - 1, -1, -1))  # pop() gives the lowest
        self._held = set()

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self, n: int = 1) -> List[int]:
        if n < 0:
            raise InvalidError(f"cannot take {n} {self.what}s")
        if n > len(self._free):
            raise CacheMemoryError(f"{n} {self.what}s wanted, {len(self._free)} free of {self.count}")
        out = [self._free.pop() for _ in range(n)]
        self._held.update(out)
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if i not in self._held:
                raise InvalidError(f"{self.what} {i} is not held (freed twice, or never taken)")
        if len(set(ids)) != len(ids):
            raise InvalidError(f"{self.what} given back twice in one call")
        for i in ids:
            self._held.remove(i)
            self._free.append(i)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return i in self._held
