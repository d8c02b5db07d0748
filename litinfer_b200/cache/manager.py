"""The cache manager: pages of keys and values, block tables, state slots.

Schedule entries whose mixers ask for the same :class:`PagedKV` (key heads,
head size, window) form a *group*.  A group has one page-id space, one pool,
one device tensor ``[entries, 2 (k|v), pages + 1, kv_heads, page_size * head_dim]``
(keys of a page as ``[page_size, head_dim]``, values transposed as
``[head_dim, page_size]``: the layout the attention kernels read without
staging) and, per request, one block table that is valid for all of its entries.
LitInfer has one pool, free list and block table per layer
(src/llaisys/models/qwen2.hpp:76-79), all identical in practice.

Pages are allocated when a request grows (``extend``), given back when it ends
(``release``) and, in a group with a window, as soon as every key on them lies
behind the window of all further queries (``commit``).  The extra last page of
each tensor is a sink for padded tokens of captured decode batches; it is
never handed out.

Mixers with :class:`FixedState` get, per owning entry, a tensor
``[max_requests + 1, *shape]``; a request holds one slot index from admission
to release, for all of them.  The slot is assigned even when no entry has
state (Qwen2 has none), and cleared at admission.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

import ctypes

from ..parts.base import FixedState, PagedKV
from . import native
from .pool import OutOfPages, PoolError, PoolView


@dataclass
class EntryCache:
    """What one schedule entry's mixer sees."""

    kind: str                               # "paged" | "state" | "none"
    writes: bool = True
    group: int = -1
    k: Optional[torch.Tensor] = None        # [pages + 1, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None        # [pages + 1, kv_heads, head_dim, page_size]
    state: Optional[torch.Tensor] = None    # [max_requests + 1, *shape]


@dataclass
class Group:
    key: PagedKV
    entries: List[int]
    pool: Optional[PoolView]
    kv: Optional[torch.Tensor]
    # the device's resident copy of the requests' block tables: int32 [max_requests + 1, table_blocks], a row per state
    # slot, the last row (the padding sequences') all sink page; a step uploads what changed (engine.batch.pack_step)
    tables: Optional[torch.Tensor] = None


class RequestCache:
    """What one live request holds.  The block tables are the host runtime's; ``tables`` reads them out."""

    __slots__ = ("request_id", "slot", "length", "_manager")

    def __init__(self, request_id: int, slot: int, manager: "CacheManager") -> None:
        self.request_id = request_id
        self.slot = slot
        self.length = 0                     # tokens whose keys and values are cached
        self._manager = manager

    @property
    def tables(self) -> List[List[int]]:
        """Per group: logical page -> page id, -1 once given back (a copy)."""
        return [self._manager.table(self, gid) for gid in range(len(self._manager.groups))]

    def num_blocks(self, group: int) -> int:
        return self._manager.table_length(self, group)

    def pages_held(self, group: int) -> List[int]:
        return [p for p in self._manager.table(self, group) if p >= 0]


class CacheManager:
    RELEASED = -1

    def __init__(self, requirements: Sequence, cache_from: Sequence[Optional[int]], num_pages: int, page_size: int,
                 max_requests: int, dtype: torch.dtype, device, allocate: bool = True, table_blocks: Optional[int] = None) -> None:
        """``table_blocks``: how many pages the longest request's table can name (default: 65,536 tokens' worth)."""
        if page_size < 16 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two of at least 16, got {page_size}")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: List[Group] = []
        self.entries: List[EntryCache] = []
        self.live: Dict[int, RequestCache] = {}
        by_key: Dict[PagedKV, int] = {}
        for i, req in enumerate(requirements):
            if cache_from[i] is not None:
                continue
            if isinstance(req, PagedKV):
                if req not in by_key:
                    by_key[req] = len(self.groups)
                    self.groups.append(Group(req, [], None, None))
                self.groups[by_key[req]].entries.append(i)
        if self.num_pages <= 0 or self.max_requests <= 0:
            raise ValueError("a cache needs at least one page and one request slot")
        # pools, block tables and the step packer live in the host runtime (csrc/host/runtime.cpp)
        self._lib = native.library()
        windows = (ctypes.c_int * max(len(self.groups), 1))(*[int(g.key.window or 0) for g in self.groups])
        self._h = self._lib.li_cm_create(len(self.groups), windows, self.num_pages, self.page_size, self.max_requests)
        if not self._h:
            raise PoolError("the host runtime could not create the cache manager")
        self.slots = PoolView(self, -1, self.max_requests)
        for gid, g in enumerate(self.groups):
            g.pool = PoolView(self, gid, self.num_pages)
        self.table_blocks = int(table_blocks or -(-65536 // self.page_size))
        for g in self.groups:
            if allocate:
                g.tables = torch.full((self.max_requests + 1, self.table_blocks), self.num_pages, dtype=torch.int32, device=self.device)
                g.kv = torch.zeros((len(g.entries), 2, self.num_pages + 1, g.key.num_kv_heads, self.page_size * g.key.head_dim),
                                   dtype=dtype, device=self.device)
        for i, req in enumerate(requirements):
            src = cache_from[i]
            if src is not None:
                owner = self.entries[src]
                self.entries.append(EntryCache(owner.kind, False, owner.group, owner.k, owner.v, owner.state))
            elif isinstance(req, PagedKV):
                gid = by_key[req]
                g = self.groups[gid]
                j = g.entries.index(i)
                shape = (self.num_pages + 1, g.key.num_kv_heads)
                k = g.kv[j, 0].view(*shape, self.page_size, g.key.head_dim) if g.kv is not None else None
                v = g.kv[j, 1].view(*shape, g.key.head_dim, self.page_size) if g.kv is not None else None
                self.entries.append(EntryCache("paged", True, gid, k, v))
            elif isinstance(req, FixedState):
                st = torch.zeros((self.max_requests + 1,) + tuple(req.shape), dtype=req.dtype, device=self.device) if allocate else None
                self.entries.append(EntryCache("state", True, state=st))
            elif req is None:
                self.entries.append(EntryCache("none"))
            else:
                raise TypeError(f"schedule entry {i}: unknown cache requirement {req!r}")

    # ------------------------------------------------------------------
    @property
    def trash_page(self) -> int:
        return self.num_pages

    @property
    def trash_slot(self) -> int:
        return self.max_requests

    def bytes_per_page(self) -> int:
        """Bytes one page id stands for, over all groups and entries."""
        esize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * 2 * g.key.num_kv_heads * self.page_size * g.key.head_dim * esize for g in self.groups)

    def __del__(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.li_cm_destroy(h)

    def num_free_pages(self, group: int = 0) -> int:
        return self._lib.li_cm_num_free(self._h, group)

    def num_free_slots(self) -> int:
        return self._lib.li_cm_num_free(self._h, -1)

    # ------------------------------------------------------------------
    def admit(self, request_id: int) -> RequestCache:
        slot = ctypes.c_int(0)
        native.check(self._lib.li_cm_admit(self._h, int(request_id), ctypes.byref(slot)))
        for e in self.entries:
            if e.kind == "state" and e.writes and e.state is not None:
                e.state[slot.value].zero_()
        rc = RequestCache(int(request_id), slot.value, self)
        self.live[rc.request_id] = rc
        return rc

    def adopt(self, request_id: int, slot: int) -> RequestCache:
        """The host runtime admitted a request by itself (its scheduler does): the picture of it here."""
        for e in self.entries:
            if e.kind == "state" and e.writes and e.state is not None:
                e.state[slot].zero_()
        rc = RequestCache(int(request_id), int(slot), self)
        self.live[rc.request_id] = rc
        return rc

    def dropped(self, rc: RequestCache) -> None:
        """The host runtime gave a request's pages and slot back by itself: forget the picture of it here."""
        if self.live.get(rc.request_id) is rc:
            del self.live[rc.request_id]
        rc.length = 0

    def table_length(self, rc: RequestCache, group: int) -> int:
        n = self._lib.li_cm_table(self._h, rc.request_id, group, None, 0)
        if n < 0:
            raise PoolError(f"request {rc.request_id} is not live")
        return n

    def table(self, rc: RequestCache, group: int) -> List[int]:
        """A copy of the request's block table in a group: logical page -> page id, -1 once given back."""
        n = self._lib.li_cm_table(self._h, rc.request_id, group, None, 0)
        if n < 0:
            return []
        out = (ctypes.c_int * max(n, 1))()
        self._lib.li_cm_table(self._h, rc.request_id, group, out, n)
        return list(out[:n])

    def pages_needed(self, rc: RequestCache, new_length: int) -> List[int]:
        need = (ctypes.c_int * max(len(self.groups), 1))()
        native.check(self._lib.li_cm_pages_needed(self._h, rc.request_id, int(new_length), need))
        return list(need[:len(self.groups)])

    def can_extend(self, rc: RequestCache, new_length: int, reserve: int = 0) -> bool:
        need = self.pages_needed(rc, new_length)
        return all(n + reserve <= self.num_free_pages(gid) or n == 0 for gid, n in enumerate(need))

    def extend(self, rc: RequestCache, new_length: int) -> None:
        """Pages for positions up to ``new_length`` in every group; all or nothing."""
        native.check(self._lib.li_cm_extend(self._h, rc.request_id, int(new_length)))

    def commit(self, rc: RequestCache, new_length: int) -> None:
        """The step has written positions below ``new_length``.  Give back the
        pages of windowed groups that no further query can read."""
        native.check(self._lib.li_cm_commit(self._h, rc.request_id, int(new_length)))
        rc.length = int(new_length)

    def commit_many(self, caches: Sequence[RequestCache], new_lengths: Sequence[int]) -> None:
        """:meth:`commit` for the requests of a step at once."""
        n = len(caches)
        ids = (ctypes.c_int * n)(*[rc.request_id for rc in caches])
        lens = (ctypes.c_int * n)(*[int(x) for x in new_lengths])
        native.check(self._lib.li_cm_commit_many(self._h, n, ids, lens))
        for rc, x in zip(caches, new_lengths):
            rc.length = int(x)

    def release(self, rc: RequestCache) -> None:
        if self.live.get(rc.request_id) is not rc:
            raise PoolError(f"request {rc.request_id} is not live")
        native.check(self._lib.li_cm_release(self._h, rc.request_id))
        rc.length = 0
        del self.live[rc.request_id]

    def slot_of(self, rc: RequestCache, group: int, position: int) -> int:
        """Flat index (page * page_size + offset) of a position in a group's pages."""
        page = self.table(rc, group)[position // self.page_size]
        if page == self.RELEASED:
            raise PoolError(f"position {position} of request {rc.request_id} lies on a page that was given back")
        return page * self.page_size + position % self.page_size

    def check(self) -> None:
        """Invariants, for tests: no page lost, held twice, or held by a dead request."""
        native.check(self._lib.li_cm_check(self._h))
        for rc in self.live.values():
            if self._lib.li_cm_length(self._h, rc.request_id) != rc.length:
                raise PoolError(f"request {rc.request_id}: length {rc.length} here, {self._lib.li_cm_length(self._h, rc.request_id)} in the host runtime")
