"""Host-side bookkeeping of one pool of pages (or slots): a LIFO free list with
ownership checks, kept by the host runtime (``csrc/host/runtime.cpp``).

LitInfer keeps one such list per layer and checks only the range of a freed
id (src/llaisys/kv_cache/block_kv_cache.hpp:34-59).  Here one list serves a
whole group of layers, page 0 comes out first as there, a page just given
back is the next one handed out (so reuse shows early in tests), and a page
can neither be freed twice nor by a request that does not hold it.
"""

from __future__ import annotations

import ctypes

from . import native
from .native import OutOfPages, PoolError

__all__ = ["OutOfPages", "PagePool", "PoolError"]


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


class PoolView:
    """One of a manager's pools (a group's pages, or the state slots), seen from outside: counts and ownership."""

    def __init__(self, manager, which: int, num_pages: int) -> None:
        self._m = manager
        self._which = which
        self.num_pages = num_pages

    @property
    def num_free(self) -> int:
        return self._m._lib.li_cm_num_free(self._m._h, self._which)

    @property
    def num_used(self) -> int:
        return self.num_pages - self.num_free

    def owner_of(self, page: int) -> int:
        return self._m._lib.li_cm_owner(self._m._h, self._which, int(page))

    def check(self) -> None:
        native.check(self._m._lib.li_cm_pool_check(self._m._h, self._which))
