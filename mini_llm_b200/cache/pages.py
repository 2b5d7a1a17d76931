"""Page allocator: a LIFO free list with an in-use flag per page.

Same role as the reference's BlockManager (src/runtime/block_manager.cu:39-99:
pop the back of the free vector, flag per block, diagnostics for an invalid id
and a double free), without its CPU half.
"""
from __future__ import annotations

from typing import Iterable, List


class PageError(RuntimeError):
    """A page id that is invalid, handed out twice or freed twice."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        # the lowest ids are handed out first
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._in_use = bytearray(num_pages)
        self.peak_in_use = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_in_use(self) -> int:
        return self.num_pages - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return 0 <= n <= len(self._free)

    def allocate(self, n: int) -> List[int]:
        """n pages, all or nothing."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise PageError(f"asked for {n} pages, {len(self._free)} free")
        if n == 0:
            return []
        out = self._free[-n:]
        out.reverse()                       # the order in which single pops would have handed them out
        in_use = self._in_use
        for p in out:
            if in_use[p]:
                raise PageError(f"page {p} was on the free list while in use")
        del self._free[-n:]
        for p in out:
            in_use[p] = 1
        self.peak_in_use = max(self.peak_in_use, self.num_in_use)
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages):
                raise PageError(f"page id {p} is outside 0..{self.num_pages - 1}")
            if not self._in_use[p]:
                raise PageError(f"page {p} freed twice")
            self._in_use[p] = 0
            self._free.append(p)

    def is_in_use(self, p: int) -> bool:
        return bool(self._in_use[p])

    def check(self) -> None:
        """Every page is either on the free list once or in use, never both."""
        seen = bytearray(self.num_pages)
        for p in self._free:
            if seen[p]:
                raise PageError(f"page {p} is on the free list twice")
            seen[p] = 1
            if self._in_use[p]:
                raise PageError(f"page {p} is free and in use")
        for p in range(self.num_pages):
            if not seen[p] and not self._in_use[p]:
                raise PageError(f"page {p} is lost: neither free nor in use")
