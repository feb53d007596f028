"""A pool of fixed-size cache pages identified by integer ids.

As in the reference's block pool (kvcore/kv/block_pool.py:71-129; kv_utils.py:108-184), id 0
is a null page that is never handed out (a table entry of 0 means "no page"), pages are
taken from the head of a free queue and returned to its tail, and a request's pages are
returned in reverse order so that tail pages are reused first.  There is no sharing between
requests here, so a page is either free or held by exactly one owner; taking or returning a
page in the wrong state raises.
"""
from __future__ import annotations

from collections import deque
from typing import Iterable

NULL_PAGE = 0


class PagePoolError(RuntimeError):
    """A page was requested that does not exist, freed twice, or freed while free."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 2:
            raise ValueError(f"a page pool needs the null page and at least one more, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: deque[int] = deque(range(1, self.num_pages))
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_usable(self) -> int:
        return self.num_pages - 1

    def usage(self) -> float:
        return 1.0 - self.num_free / self.num_usable

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError(f"cannot allocate {count} pages")
        if count > len(self._free):
            raise PagePoolError(f"asked for {count} pages but only {len(self._free)} are free")
        pages = [self._free.popleft() for _ in range(count)]
        for page in pages:
            self._held[page] = True
        return pages

    def free(self, pages: Iterable[int]) -> None:
        for page in pages:
            if page == NULL_PAGE:
                raise PagePoolError("the null page cannot be freed")
            if not 0 < page < self.num_pages:
                raise PagePoolError(f"page {page} does not exist in a pool of {self.num_pages}")
            if not self._held[page]:
                raise PagePoolError(f"page {page} is freed twice")
            self._held[page] = False
            self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def free_pages(self) -> list[int]:
        return list(self._free)


__all__ = ["NULL_PAGE", "PagePool", "PagePoolError"]
