"""The host runtime's pool on its own (``li_pool_*`` in csrc/host/runtime.cpp) behind a small class, for the tests of its
invariants; the engine reaches its pools through the cache manager."""

from __future__ import annotations

import ctypes

from litinfer_b200.cache import native
from litinfer_b200.cache.native import PoolError


class PagePool:
    FREE = -1

    def __init__(self, num_pages: int, what: str = "page") -> None:
        if num_pages <= 0:
            raise ValueError(f"a pool needs at least one {what}")
        self.num_pages = int(num_pages)
        self.what = what
        self._lib = native.library()
        self._h = self._lib.li_pool_create(self.num_pages, what.encode())
        if not self._h:
            raise PoolError(f"cannot create a pool of {num_pages} {what}s")

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.li_pool_destroy(h)

    @property
    def num_free(self) -> int:
        return self._lib.li_pool_num_free(self._h)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    def owner_of(self, page: int) -> int:
        return self._lib.li_pool_owner(self._h, int(page))

    def alloc(self, owner: int) -> int:
        page = ctypes.c_int(0)
        native.check(self._lib.li_pool_alloc(self._h, int(owner), ctypes.byref(page)))
        return page.value

    def free(self, page: int, owner: int) -> None:
        native.check(self._lib.li_pool_free(self._h, int(page), int(owner)))

    def check(self) -> None:
        """Every page is either free exactly once or owned, never both."""
        native.check(self._lib.li_pool_check(self._h))
