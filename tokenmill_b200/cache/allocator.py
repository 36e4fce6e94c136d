"""Page allocator: a free stack, reference counts, and (with prefix caching) a least-recently-used
list of pages whose content may still be revived.

Behaviour kept from the reference's BlockAllocator (src/infer/kv/block_allocator.py:19-87): a page
has a reference count; counts above one come from requests sharing a cached prefix; a released page
that holds a published (hashed) prefix is parked as evictable instead of free, can be revived by
``share``, and is evicted, oldest first, only when the free list is empty. Asking for more pages than
are available raises ``OutOfPages`` and changes nothing. Differences: the free list is a stack (the
page released last is handed out first, so recently used memory is reused while it is still in the
L2 cache) and every misuse raises instead of asserting.
"""

from __future__ import annotations

from collections import OrderedDict
from collections.abc import Callable


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int, enable_caching: bool = False,
                 on_evict: Callable[[int], None] | None = None):
        if num_pages < 1:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: list[int] = list(range(num_pages - 1, -1, -1))     # stack; page 0 comes out first
        self.refcount = [0] * num_pages
        self.enable_caching = enable_caching
        self._evictable: OrderedDict[int, None] = OrderedDict()          # refcount 0, content published
        self._cached: set[int] = set()
        self._on_evict = on_evict

    @property
    def num_free(self) -> int:
        """Pages ``allocate`` can hand out now (free + evictable)."""
        return len(self._free) + len(self._evictable)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    def allocate(self, n: int) -> list[int]:
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > self.num_free:
            raise OutOfPages(f"need {n} pages, {self.num_free} available")
        out = []
        for _ in range(n):
            if self._free:
                page = self._free.pop()
            else:
                page, _ = self._evictable.popitem(last=False)            # least recently released
                self._cached.discard(page)
                if self._on_evict:
                    self._on_evict(page)
            if self.refcount[page] != 0:
                raise RuntimeError(f"page {page} handed out while still referenced")
            self.refcount[page] = 1
            out.append(page)
        return out

    def release(self, pages: list[int]) -> None:
        for page in pages:
            if not (0 <= page < self.num_pages):
                raise RuntimeError(f"page {page} is not in the pool")
            if self.refcount[page] <= 0:
                raise RuntimeError(f"double free of page {page}")
            self.refcount[page] -= 1
            if self.refcount[page] == 0:
                if self.enable_caching and page in self._cached:
                    self._evictable[page] = None
                else:
                    self._free.append(page)

    def mark_cached(self, page: int) -> None:
        if self.refcount[page] <= 0:
            raise RuntimeError(f"page {page} is not held; only a held page can be published")
        self._cached.add(page)

    def is_cached(self, page: int) -> bool:
        return page in self._cached

    def share(self, page: int) -> None:
        """Take one more reference to a published page, reviving it if it was evictable."""
        if self.refcount[page] == 0:
            if page not in self._evictable:
                raise RuntimeError(f"page {page} is free, not cached")
            del self._evictable[page]
        self.refcount[page] += 1

    def check_invariants(self) -> None:
        free, evict = set(self._free), set(self._evictable)
        if len(free) != len(self._free):
            raise AssertionError("a page is in the free list twice")
        if free & evict:
            raise AssertionError("a page is both free and evictable")
        for page in range(self.num_pages):
            pooled = page in free or page in evict
            if (self.refcount[page] == 0) != pooled:
                raise AssertionError(f"page {page}: refcount {self.refcount[page]}, in a list: {pooled}")
            if page in evict and page not in self._cached:
                raise AssertionError(f"page {page} is evictable but not published")
        if self.num_free + sum(1 for r in self.refcount if r > 0) != self.num_pages:
            raise AssertionError("free + held != total")
