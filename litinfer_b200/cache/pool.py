"""Host-side bookkeeping of one pool of pages (or slots): a LIFO free list with
ownership checks.

LitInfer keeps one such list per layer and checks only the range of a freed
id (src/llaisys/kv_cache/block_kv_cache.hpp:34-59).  Here one list serves a
whole group of layers, page 0 comes out first as there, a page just given
back is the next one handed out (so reuse shows early in tests), and a page
can neither be freed twice nor by a request that does not hold it.
"""

from __future__ import annotations

from typing import List


class PoolError(RuntimeError):
    pass


class OutOfPages(PoolError):
    pass


class PagePool:
    FREE = -1

    def __init__(self, num_pages: int, what: str = "page") -> None:
        if num_pages <= 0:
            raise ValueError(f"a pool needs at least one {what}")
        self.num_pages = int(num_pages)
        self.what = what
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._owner: List[int] = [self.FREE] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def owner_of(self, page: int) -> int:
        return self._owner[page]

    def alloc(self, owner: int) -> int:
        if owner < 0:
            raise PoolError("owner ids are non-negative")
        if not self._free:
            raise OutOfPages(f"no free {self.what} (all {self.num_pages} in use)")
        page = self._free.pop()
        self._owner[page] = owner
        return page

    def free(self, page: int, owner: int) -> None:
        if not 0 <= page < self.num_pages:
            raise PoolError(f"{self.what} {page} is outside the pool of {self.num_pages}")
        held_by = self._owner[page]
        if held_by == self.FREE:
            raise PoolError(f"{self.what} {page} freed twice")
        if held_by != owner:
            raise PoolError(f"{self.what} {page} is held by {held_by}, not by {owner}")
        self._owner[page] = self.FREE
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free exactly once or owned, never both."""
        seen = set()
        for p in self._free:
            if p in seen:
                raise PoolError(f"{self.what} {p} is on the free list twice")
            if self._owner[p] != self.FREE:
                raise PoolError(f"{self.what} {p} is free and owned by {self._owner[p]}")
            seen.add(p)
        for p, o in enumerate(self._owner):
            if o == self.FREE and p not in seen:
                raise PoolError(f"{self.what} {p} is lost: neither free nor owned")
