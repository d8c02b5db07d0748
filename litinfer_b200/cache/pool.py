"""Host-side bookkeeping of the pools of pages (and slots): LIFO free lists with
ownership checks, kept by the host runtime (``csrc/host/runtime.cpp``); here the view of one of a
manager's pools.  (The runtime's pool on its own, ``li_pool_*``, is driven by the tests: tests/pool_face.py.)

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

__all__ = ["OutOfPages", "PoolError", "PoolView"]


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
