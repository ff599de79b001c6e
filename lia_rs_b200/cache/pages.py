"""Host bookkeeping of one pool of fixed-size pages: a free list and a user count per page.

The reference keeps `users` per page and refuses an underflow (src/inference/page_cache.rs:12-16,
240-245).  Pages are handed out from a LIFO free list, so a page that was just given back is the
next to be used again.  A user count above one is reserved for sharing pages between requests
(the reference's prefix cache attaches there; it is not built here)."""
from __future__ import annotations


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise PageError("empty page pool")
        self.num_pages = int(num_pages)
        self._free = list(range(self.num_pages - 1, -1, -1))     # pop() yields page 0 first
        self._users = [0] * self.num_pages

    def available(self) -> int:
        return len(self._free)

    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise PageError("page pool exhausted")
        page = self._free.pop()
        if self._users[page] != 0:
            raise PageError(f"page {page} on the free list is held")
        self._users[page] = 1
        return page

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise PageError(f"page {page} is outside the pool")
        if self._users[page] <= 0:
            raise PageError(f"page {page} freed twice")
        self._users[page] -= 1
        if self._users[page] == 0:
            self._free.append(page)

    def users(self, page: int) -> int:
        return self._users[page]

    def check(self, held_pages) -> None:
        """Invariant: every page is either on the free list once or held by exactly the given
        holders.  `held_pages` lists the pages that the block tables hold (with repetition)."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageError("a page is on the free list twice")
        counts = {}
        for page in held_pages:
            counts[page] = counts.get(page, 0) + 1
        for page in range(self.num_pages):
            expected = counts.get(page, 0)
            if self._users[page] != expected:
                raise PageError(f"page {page}: {self._users[page]} users recorded, {expected} holders found")
            if (expected == 0) != (page in free):
                raise PageError(f"page {page} is lost or both held and free")
