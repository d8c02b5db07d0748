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

from ..parts.base import FixedState, PagedKV
from .pool import OutOfPages, PagePool, PoolError


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
    pool: PagePool
    kv: Optional[torch.Tensor]


@dataclass
class RequestCache:
    """What one live request holds."""

    request_id: int
    slot: int
    length: int = 0                         # tokens whose keys and values are cached
    tables: List[List[int]] = field(default_factory=list)   # per group: logical page -> page id, -1 once given back

    def pages_held(self, group: int) -> List[int]:
        return [p for p in self.tables[group] if p >= 0]


class CacheManager:
    RELEASED = -1

    def __init__(self, requirements: Sequence, cache_from: Sequence[Optional[int]], num_pages: int, page_size: int,
                 max_requests: int, dtype: torch.dtype, device, allocate: bool = True) -> None:
        if page_size < 16 or page_size & (page_size - 1):
            raise ValueError(f"page_size must be a power of two of at least 16, got {page_size}")
        self.page_size = int(page_size)
        self.num_pages = int(num_pages)
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: List[Group] = []
        self.entries: List[EntryCache] = []
        self.slots = PagePool(self.max_requests, "state slot")
        self.live: Dict[int, RequestCache] = {}
        by_key: Dict[PagedKV, int] = {}
        for i, req in enumerate(requirements):
            if cache_from[i] is not None:
                continue
            if isinstance(req, PagedKV):
                if req not in by_key:
                    by_key[req] = len(self.groups)
                    self.groups.append(Group(req, [], PagePool(self.num_pages), None))
                self.groups[by_key[req]].entries.append(i)
        for g in self.groups:
            if allocate:
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

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def num_free_slots(self) -> int:
        return self.slots.num_free

    # ------------------------------------------------------------------
    def admit(self, request_id: int) -> RequestCache:
        if request_id in self.live:
            raise PoolError(f"request {request_id} is already admitted")
        slot = self.slots.alloc(request_id)
        for e in self.entries:
            if e.kind == "state" and e.writes and e.state is not None:
                e.state[slot].zero_()
        rc = RequestCache(request_id, slot, 0, [[] for _ in self.groups])
        self.live[request_id] = rc
        return rc

    def _first_needed_page(self, g: Group, length: int) -> int:
        """First logical page that a query at position >= ``length`` can still read."""
        if g.key.window is None:
            return 0
        first_key = max(0, length - g.key.window + 1)
        return first_key // self.page_size

    def pages_needed(self, rc: RequestCache, new_length: int) -> List[int]:
        want = -(-new_length // self.page_size)
        return [max(0, want - len(rc.tables[gid])) for gid in range(len(self.groups))]

    def can_extend(self, rc: RequestCache, new_length: int, reserve: int = 0) -> bool:
        need = self.pages_needed(rc, new_length)
        return all(n + reserve <= g.pool.num_free or n == 0 for n, g in zip(need, self.groups))

    def extend(self, rc: RequestCache, new_length: int) -> None:
        """Pages for positions up to ``new_length`` in every group; all or nothing."""
        need = self.pages_needed(rc, new_length)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {rc.request_id} needs {n} pages, {g.pool.num_free} are free")
        for gid, (n, g) in enumerate(zip(need, self.groups)):
            for _ in range(n):
                rc.tables[gid].append(g.pool.alloc(rc.request_id))

    def commit(self, rc: RequestCache, new_length: int) -> None:
        """The step has written positions below ``new_length``.  Give back the
        pages of windowed groups that no further query can read."""
        if new_length < rc.length:
            raise PoolError("a request's length never shrinks")
        rc.length = new_length
        for gid, g in enumerate(self.groups):
            if g.key.window is None:
                continue
            table = rc.tables[gid]
            for lp in range(min(self._first_needed_page(g, new_length), len(table))):
                if table[lp] != self.RELEASED:
                    g.pool.free(table[lp], rc.request_id)
                    table[lp] = self.RELEASED

    def release(self, rc: RequestCache) -> None:
        if self.live.get(rc.request_id) is not rc:
            raise PoolError(f"request {rc.request_id} is not live")
        for gid, g in enumerate(self.groups):
            # last page first, so that a request admitted next gets them in ascending order
            for p in reversed(rc.tables[gid]):
                if p != self.RELEASED:
                    g.pool.free(p, rc.request_id)
            rc.tables[gid] = []
        self.slots.free(rc.slot, rc.request_id)
        rc.length = 0
        del self.live[rc.request_id]

    def slot_of(self, rc: RequestCache, group: int, position: int) -> int:
        """Flat index (page * page_size + offset) of a position in a group's pages."""
        page = rc.tables[group][position // self.page_size]
        if page == self.RELEASED:
            raise PoolError(f"position {position} of request {rc.request_id} lies on a page that was given back")
        return page * self.page_size + position % self.page_size

    def check(self) -> None:
        """Invariants, for tests: no page lost, held twice, or held by a dead request."""
        self.slots.check()
        for gid, g in enumerate(self.groups):
            g.pool.check()
            held = {}
            for rc in self.live.values():
                for p in rc.pages_held(gid):
                    if p in held:
                        raise PoolError(f"page {p} of group {gid} is held by requests {held[p]} and {rc.request_id}")
                    held[p] = rc.request_id
                    if g.pool.owner_of(p) != rc.request_id:
                        raise PoolError(f"page {p} of group {gid}: table of {rc.request_id}, pool says {g.pool.owner_of(p)}")
            if len(held) != g.pool.num_used:
                raise PoolError(f"group {gid}: {g.pool.num_used} pages in use, {len(held)} in block tables")
