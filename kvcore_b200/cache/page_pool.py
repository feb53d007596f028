"""A pool of fixed-size cache pages identified by integer ids.

As in the reference's block pool (kvcore/kv/block_pool.py:71-129, 196-207; kv_utils.py:71-184),
id 0 is a null page that is never handed out (a table entry of 0 means "no page"), pages are
taken from the head of a free queue and returned to its tail, and a request's pages are
returned in reverse order so that tail pages are reused first.  A page carries a reference
count: normally one owner; with prefix reuse several requests may hold the same page, and a
page whose contents are registered under a key stays findable after its last owner let go of
it, until the queue hands it out again (then the key is dropped).  Taking or returning a page
in the wrong state raises.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Hashable, Iterable

NULL_PAGE = 0


class PagePoolError(RuntimeError):
    """A page was requested that does not exist, freed twice, or freed while free."""


class PagePool:
    def __init__(self, num_pages: int) -> None:
        if num_pages < 2:
            raise ValueError(f"a page pool needs the null page and at least one more, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: OrderedDict[int, None] = OrderedDict((page, None) for page in range(1, self.num_pages))
        self._refs = [0] * self.num_pages
        self._key_of: dict[int, Hashable] = {}
        self._page_of: dict[Hashable, int] = {}

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
        pages = []
        for _ in range(count):
            page, _ = self._free.popitem(last=False)
            key = self._key_of.pop(page, None)
            if key is not None:          # its old contents are about to be overwritten
                del self._page_of[key]
            self._refs[page] = 1
            pages.append(page)
        return pages

    def free(self, pages: Iterable[int]) -> None:
        """Drop one reference of each page; a page nobody holds goes to the tail of the queue."""
        for page in pages:
            if page == NULL_PAGE:
                raise PagePoolError("the null page cannot be freed")
            if not 0 < page < self.num_pages:
                raise PagePoolError(f"page {page} does not exist in a pool of {self.num_pages}")
            if self._refs[page] <= 0:
                raise PagePoolError(f"page {page} is freed twice")
            self._refs[page] -= 1
            if self._refs[page] == 0:
                self._free[page] = None

    def is_held(self, page: int) -> bool:
        return self._refs[page] > 0

    def ref_count(self, page: int) -> int:
        return self._refs[page]

    def free_pages(self) -> list[int]:
        return list(self._free)

    # ---- reuse of registered contents ----------------------------------------------------------
    def register(self, page: int, key: Hashable) -> bool:
        """Make the contents of a held page findable under ``key``.  False if the key is taken."""
        if self._refs[page] <= 0:
            raise PagePoolError(f"page {page} is not held and cannot be registered")
        if key in self._page_of or page in self._key_of:
            return False
        self._key_of[page] = key
        self._page_of[key] = page
        return True

    def lookup(self, key: Hashable) -> int | None:
        return self._page_of.get(key)

    def is_queued(self, page: int) -> bool:
        """Whether the page sits in the free queue (held by nobody, contents possibly findable)."""
        return page in self._free

    def share(self, page: int) -> None:
        """Take one more reference of a page found by ``lookup`` (out of the queue if nobody held it)."""
        if not 0 < page < self.num_pages or page not in self._key_of:
            raise PagePoolError(f"page {page} has no registered contents to share")
        if self._refs[page] == 0:
            del self._free[page]
        self._refs[page] += 1


__all__ = ["NULL_PAGE", "PagePool", "PagePoolError"]
