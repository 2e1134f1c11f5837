"""Host-side bookkeeping of the cache: who holds which slot and which pages.

Pure Python, no tensors: the tests of "no slot lost, held twice or freed twice"
run on these classes alone. The reference has nothing of the kind: its batch
row is the slot, fixed for a plan, and "reset" is ``pos.zero_()``
(engine/model.py:231-234,290 of willzeng274/kernel-rush-kawk).
"""

from __future__ import annotations


class CacheError(RuntimeError):
    """No free slot or page, a slot used that is not held, or a sequence longer
    than the cache was built for."""


class FreeList:
    """Integers 0..n-1, handed out and taken back. Last freed, first reused, so that
    reuse is exercised at once rather than after a full cycle."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))
        self._held = [False] * n

    def __len__(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.n} are held")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice, or was never handed out")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Every index is either free exactly once or held; raises otherwise."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise CacheError(f"a {self.what} sits in the free list twice")
        for i in range(self.n):
            if self._held[i] == (i in seen):
                raise CacheError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")


class PageLedger:
    """Pages of one storage group: a pool and, per slot, the pages it holds in
    logical order. ``ring`` is None for a group that keeps every position, or the
    number of logical pages a slot cycles through for a group that keeps a window."""

    def __init__(self, n_pages: int, n_slots: int, width: int, page_size: int, ring: int | None):
        self.pool = FreeList(n_pages, "cache page")
        self.pages: list[list[int]] = [[] for _ in range(n_slots)]
        self.width = width
        self.page_size = page_size
        self.ring = ring

    def pages_for(self, length: int) -> int:
        need = -(-length // self.page_size)
        return min(need, self.ring) if self.ring is not None else need

    def can_grow(self, slot: int, length: int) -> bool:
        return self.pages_for(length) - len(self.pages[slot]) <= len(self.pool)

    def grow(self, slot: int, length: int) -> list[tuple[int, int]]:
        """Make ``slot`` hold pages for ``length`` tokens; returns the new (logical
        index, page) pairs."""
        need = self.pages_for(length)
        if need > self.width:
            raise CacheError(f"a sequence of {length} tokens needs {need} pages; the cache was built for {self.width} "
                             f"({self.width * self.page_size} tokens a sequence)")
        have = self.pages[slot]
        if need - len(have) > len(self.pool):
            raise CacheError(f"the cache is full: {need - len(have)} more pages of {self.page_size} tokens are needed, "
                             f"{len(self.pool)} of {self.pool.n} are free")
        new = []
        while len(have) < need:
            page = self.pool.take()
            new.append((len(have), page))
            have.append(page)
        return new

    def release(self, slot: int) -> None:
        for page in self.pages[slot]:
            self.pool.give(page)
        self.pages[slot] = []

    def check(self) -> None:
        self.pool.check()
        held = [p for pages in self.pages for p in pages]
        if len(held) != len(set(held)):
            raise CacheError("a cache page is held by two slots")
        if len(held) != self.pool.held:
            raise CacheError(f"{self.pool.held} pages are handed out but slots hold {len(held)}")
