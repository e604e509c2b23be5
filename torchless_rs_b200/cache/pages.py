"""Free lists with ownership checks, for cache pages and for sequence slots.

The reference keeps one tensor [layers, kv heads, max_seq_len, head_dim] for the keys and one for the
values of its single sequence (src/model/kv_cache.rs:23-53); pages and slots take its place for
batches of sequences that come and go."""
from __future__ import annotations

from typing import List


class CacheCapacityError(RuntimeError):
    """The cache has no room for what a step needs."""


class CacheStateError(RuntimeError):
    """A slot or page was released twice or used without being held."""


class CacheRollbackError(RuntimeError):
    """A sequence cannot be shortened to the asked length: a window has already given back
    keys that the shorter sequence's next position would see, or a mixer keeps state of fixed
    size, which holds no record of earlier lengths."""


class FreeList:
    """Integers 0..n-1 handed out lowest first; an item is either free or held,
    never both, and never lost."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))  # pop() gives the lowest
        self._held = [False] * n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self, count: int = 1) -> List[int]:
        if count > len(self._free):
            raise CacheCapacityError(
                f"out of {self.what}s: {count} wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, items) -> None:
        items = list(items)
        for i in items:
            if not 0 <= i < self.n:
                raise CacheStateError(f"{self.what} {i} does not exist")
            if not self._held[i]:
                raise CacheStateError(f"{self.what} {i} is given back but is not held")
            self._held[i] = False
        self._free.extend(sorted(items, reverse=True))
        # keep lowest-first order so reuse is deterministic
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every item is in exactly one of the two states."""
        if len(set(self._free)) != len(self._free):
            raise CacheStateError(f"a {self.what} is in the free list twice")
        for i in self._free:
            if self._held[i]:
                raise CacheStateError(f"{self.what} {i} is both free and held")
        if sum(self._held) + len(self._free) != self.n:
            raise CacheStateError(f"a {self.what} was lost")
