"""Page allocator: a fixed set of page ids and a LIFO free list.

cklxx/arle keeps the same structure inside its token pool: a stack of free page
ids initialised so that page 0 is handed out first, growth that fails without
changing anything (crates/cuda-kernels/src/paged_kv.rs:416, :498-533).  Its
reference counts exist for a prefix cache, which this engine does not have; here
a page has exactly one holder or is free, and the allocator checks that.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Raised by an allocation that does not fit; nothing has been changed."""

    def __init__(self, wanted: int, free: int, what: str = "pages"):
        super().__init__(f"out of {what}: wanted {wanted}, {free} free")
        self.wanted, self.free = wanted, free


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives 0 first
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("negative page count")
        if n > len(self._free):
            raise OutOfPages(n, len(self._free))
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._held[p] = 1
        return pages

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise RuntimeError(f"page {p} freed twice")
            self._held[p] = 0
            self._free.append(p)

    def check(self) -> None:
        """Every page is free exactly once or held exactly once."""
        seen = bytearray(self.num_pages)
        for p in self._free:
            if seen[p]:
                raise AssertionError(f"page {p} is on the free list twice")
            seen[p] = 1
            if self._held[p]:
                raise AssertionError(f"page {p} is both free and held")
        if sum(seen) + sum(self._held) != self.num_pages:
            raise AssertionError("a page is neither free nor held")
