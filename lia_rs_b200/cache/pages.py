"""Host bookkeeping of one pool of fixed-size pages: a free list and a user count per page.

The reference keeps `users` per page and refuses an underflow (src/inference/page_cache.rs:12-16,
240-245).  Pages are handed out from a LIFO free list, so a page that was just given back is the
next to be used again.  A user count above one is reserved for sharing pages between requests
(the reference's prefix cache attaches there; it is not built here).

The state lives in the native host library (csrc/host/cache_host.cpp); this class is its face."""
from __future__ import annotations

import ctypes

from ..kernels import build


class PageError(RuntimeError):
    pass


def host_library():
    return build.load_host()


def raise_last(default: str = "the cache's host library refused"):
    message = host_library().lia_host_error()
    raise PageError(message.decode() if message else default)


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise PageError("empty page pool")
        self.num_pages = int(num_pages)
        self._lib = host_library()
        self._handle = ctypes.c_void_p(self._lib.lia_pool_create(self.num_pages))
        if not self._handle:
            raise_last()

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.lia_pool_destroy(handle)

    def available(self) -> int:
        return self._lib.lia_pool_available(self._handle)

    def in_use(self) -> int:
        return self.num_pages - self.available()

    def allocate(self) -> int:
        page = self._lib.lia_pool_allocate(self._handle)
        if page < 0:
            raise_last()
        return page

    def release(self, page: int) -> None:
        if self._lib.lia_pool_release(self._handle, int(page)) < 0:
            raise_last()

    def users(self, page: int) -> int:
        return self._lib.lia_pool_users(self._handle, int(page))

    def check(self, held_pages) -> None:
        """Invariant: every page is either on the free list once or held by exactly the given
        holders.  `held_pages` lists the pages that the block tables hold (with repetition)."""
        held = list(held_pages)
        array = (ctypes.c_int * max(1, len(held)))(*held)
        if self._lib.lia_pool_check(self._handle, array, len(held)) < 0:
            raise_last()
