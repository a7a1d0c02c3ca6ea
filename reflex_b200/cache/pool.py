"""Free lists of the cache: slots (one per live sequence) and pages.

Pure host bookkeeping, no tensors.  Every id is either free or held, never
both; giving back an id that is not held, or asking for more than is free, is
an error and changes nothing.
"""

from __future__ import annotations

from typing import Iterable, List

from ..errors import CacheError, OutOfMemory


class IdPool:
    def __init__(self, count: int, what: str):
        if count < 0:
            raise ValueError("count must be >= 0")
        self.what = what
        self.count = count
        # a stack with the lowest id on top: freed ids are handed out again first
        self._free: List[int] = list(range(count - 1, -1, -1))
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.count and self._held[i]

    def take(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError("n must be >= 0")
        if n > len(self._free):
            raise OutOfMemory(
                f"cache is out of {self.what}s: {n} wanted, {len(self._free)} of {self.count} free"
            )
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._held[i] = True
        return out

    def give(self, ids: Iterable[int]) -> None:
        ids = list(ids)
        seen = set()
        for i in ids:
            if not (0 <= i < self.count) or not self._held[i] or i in seen:
                raise CacheError(f"{self.what} {i} is not held (freed twice or never taken)")
            seen.add(i)
        for i in ids:
            self._held[i] = False
            self._free.append(i)
