"""The cache manager: keys and values in pages with a block table per request, and slots of fixed-size
per-request state.

Sites (entries of a model's run order) declare what they need (`PagedNeed`, `SlotNeed`). Sites whose
paged needs agree (KV heads, head size, window) form a *group*: one pool of page ids and one block table
per request, each site with K and V tensors of its own indexed by the same page ids. Groups with
different needs (all keys; a window of them) have pools of their own. A request holds
ceil(length / page_size) pages of every group (fewer for a windowed group: pages the window has passed
are given back as the request advances), and one state slot. Pages and the slot return when the request
ends; freed pages are handed out again last-freed-first, so reuse happens at once.

The reference keeps the same split between position-indexed "views" (K, V) and fixed-size "sections"
(conv states) of a sequence's cache (engine/models/state.py:36-83) and pages its K/V through a pool with
one byte account and a `PoolFull` error (engine/kvpool.py:204-345); here pages are rows of preallocated
tensors, named by a block table, instead of mapped virtual memory.

The bookkeeping is plain Python and needs no device: with `device=None` no tensor is made.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import PagedNeed, PagedSiteCache, SlotNeed, SlotSiteCache


class OutOfPages(RuntimeError):
    """A reservation needs more pages (or a slot) than are free; nothing was taken."""


class PagePool:
    """Page ids 0..n-1 with a free list. A page is free or held by exactly one owner."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))     # pop() takes from the end: page 0 first, then LIFO reuse
        self._owner: list[object | None] = [None] * num_pages
        self.peak_used = 0
        self.reused = 0
        self._ever_used = [False] * num_pages

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int, owner) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        out = []
        for _ in range(n):
            p = self._free.pop()
            assert self._owner[p] is None, f"page {p} handed out while held by {self._owner[p]!r}"
            self._owner[p] = owner
            self.reused += self._ever_used[p]
            self._ever_used[p] = True
            out.append(p)
        self.peak_used = max(self.peak_used, self.used)
        return out

    def give_back(self, pages: list[int], owner) -> None:
        for p in pages:
            if self._owner[p] is not owner and self._owner[p] != owner:
                raise RuntimeError(f"page {p} given back by {owner!r} but held by {self._owner[p]!r}")
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]


@dataclass
class PageGroup:
    need: PagedNeed
    sites: list[int]
    pool: PagePool
    page_size: int
    tables: dict = field(default_factory=dict)      # request id -> list of page ids by page index (-1: given back)
    arrays: dict = field(default_factory=dict)      # request id -> the same table as an int32 array with room to grow
                                                    # (what a step copies to the device without walking a list)

    def extend(self, req, pages: list[int]) -> None:
        table = self.tables[req]
        arr = self.arrays[req]
        n = len(table)
        if n + len(pages) > arr.shape[0]:
            grown = np.empty(max(2 * arr.shape[0], n + len(pages)), dtype=np.int32)
            grown[:n] = arr[:n]
            arr = self.arrays[req] = grown
        arr[n:n + len(pages)] = pages
        table.extend(pages)

    def pages_needed(self, req, new_len: int) -> int:
        table = self.tables.get(req, [])
        return max(0, -(-new_len // self.page_size) - len(table))


class CacheManager:
    def __init__(self, needs: list, num_pages: int, max_requests: int, page_size: int = 16,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        """`needs[i]` is the need of site i (None: the site has no cache of its own). `num_pages` pages of
        `page_size` tokens are made for every paged group."""
        if page_size <= 0 or page_size % 16:
            raise ValueError(f"page size {page_size}: a positive multiple of 16")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, device
        self.groups: list[PageGroup] = []
        self.site_cache: list = [None] * len(needs)
        self._slot_sites: list[int] = []
        by_need: dict[PagedNeed, PageGroup] = {}
        for i, need in enumerate(needs):
            if isinstance(need, PagedNeed):
                if need.window is not None and need.window <= 0:
                    raise ValueError(f"site {i}: window {need.window} must be positive")
                if need not in by_need:
                    by_need[need] = PageGroup(need, [], PagePool(num_pages), page_size)
                    self.groups.append(by_need[need])
                by_need[need].sites.append(i)
            elif isinstance(need, SlotNeed):
                self._slot_sites.append(i)
            elif need is not None:
                raise TypeError(f"site {i}: unknown cache need {need!r}")
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self._slot_of: dict = {}
        self._length: dict = {}
        self.preemptions = 0
        self._slot_init: dict[int, object] = {}       # site -> what a slot is set to when a request takes it
        if device is not None:
            for gi, g in enumerate(self.groups):
                shape = (num_pages, g.need.kv_heads, page_size, g.need.head_dim)
                for i in g.sites:
                    self.site_cache[i] = PagedSiteCache(gi, page_size, torch.zeros(shape, dtype=dtype, device=device),
                                                        torch.zeros(shape, dtype=dtype, device=device))
            for i in self._slot_sites:
                need = needs[i]
                self.site_cache[i] = SlotSiteCache(torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=device))
                init = need.init
                if isinstance(init, torch.Tensor):
                    init = init.to(device=device, dtype=need.dtype)
                self._slot_init[i] = init

    # ---- requests ----
    def admit(self, req) -> int:
        """Give `req` a state slot (set to its site's initial value: zeros unless the need says otherwise) and empty
        block tables; returns the slot."""
        if req in self._slot_of:
            raise RuntimeError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise OutOfPages(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._slot_of[req] = slot
        self._length[req] = 0
        for g in self.groups:
            g.tables[req] = []
            g.arrays[req] = np.empty(64, dtype=np.int32)
        if self.device is not None:
            for i in self._slot_sites:
                init = self._slot_init.get(i)
                if init is None:
                    self.site_cache[i].state[slot].zero_()
                elif isinstance(init, torch.Tensor):
                    self.site_cache[i].state[slot].copy_(init.expand_as(self.site_cache[i].state[slot]))
                else:
                    self.site_cache[i].state[slot].fill_(init)
        return slot

    def has(self, req) -> bool:
        return req in self._slot_of

    def slot_of(self, req) -> int:
        return self._slot_of[req]

    def length_of(self, req) -> int:
        return self._length[req]

    def can_reserve(self, wants: list[tuple[object, int]]) -> bool:
        """Whether every (request, new length) of `wants` can be reserved together."""
        for g in self.groups:
            if sum(g.pages_needed(req, n) for req, n in wants) > g.pool.free:
                return False
        return True

    def reserve(self, req, new_len: int) -> None:
        """Make sure `req` holds pages for positions < new_len in every group; all or nothing."""
        if req not in self._slot_of:
            raise RuntimeError(f"request {req!r} is not admitted")
        for g in self.groups:
            need = g.pages_needed(req, new_len)
            if need > g.pool.free:
                raise OutOfPages(f"request {req!r} needs {need} more pages for {new_len} tokens, {g.pool.free} free "
                                 f"of {g.pool.num_pages}")
        for g in self.groups:
            need = g.pages_needed(req, new_len)
            if need:
                g.extend(req, g.pool.take(need, req))

    def advance(self, req, new_len: int) -> None:
        """The request now holds `new_len` tokens: windowed groups give back the pages no later row can read."""
        self._length[req] = new_len
        for g in self.groups:
            w = g.need.window
            if w is None:
                continue
            # the next row sits at position new_len and reads positions >= new_len - w + 1
            first_needed = max(0, new_len - w + 1) // g.page_size
            table = g.tables[req]
            gone = [p for p in table[:first_needed] if p >= 0]
            if gone:
                g.pool.give_back(gone, req)
                for j in range(min(first_needed, len(table))):
                    table[j] = -1
                g.arrays[req][:min(first_needed, len(table))] = -1

    def free(self, req) -> None:
        """The request ends (or is preempted): every page and the slot go back."""
        if req not in self._slot_of:
            raise RuntimeError(f"request {req!r} is not admitted (freed twice?)")
        for g in self.groups:
            g.pool.give_back([p for p in g.tables.pop(req) if p >= 0], req)
            del g.arrays[req]
        self._free_slots.append(self._slot_of.pop(req))
        del self._length[req]

    # ---- what a step reads ----
    def table(self, group: int, req) -> list[int]:
        return self.groups[group].tables[req]

    def table_array(self, group: int, req) -> "np.ndarray":
        """The block table of `req` in `group` as an int32 array (a view: valid until the table next grows)."""
        g = self.groups[group]
        return g.arrays[req][:len(g.tables[req])]

    def max_table_len(self, reqs) -> int:
        return max((len(g.tables[r]) for g in self.groups for r in reqs), default=0)

    def stats(self) -> dict:
        return {
            "page_size": self.page_size,
            "requests": len(self._slot_of),
            "free_slots": len(self._free_slots),
            "groups": [{"sites": len(g.sites), "window": g.need.window, "pages": g.pool.num_pages, "free": g.pool.free,
                        "peak_used": g.pool.peak_used, "reused": g.pool.reused} for g in self.groups],
        }

    def check(self) -> None:
        """Invariants: no page lost, none held twice, every table entry owned by its request."""
        for g in self.groups:
            held = [p for t in g.tables.values() for p in t if p >= 0]
            assert len(held) == len(set(held)), "a page is in two block tables"
            assert len(held) + g.pool.free == g.pool.num_pages, "a page was lost"
            assert len(set(g.pool._free)) == len(g.pool._free), "a page is on the free list twice"
            for req, t in g.tables.items():
                assert g.arrays[req][:len(t)].tolist() == t, f"the array of {req!r}'s table differs from the table"
            for req, t in g.tables.items():
                for p in t:
                    assert p < 0 or g.pool.owner_of(p) == req, f"page {p} in the table of {req!r} is held by someone else"
        assert len(self._free_slots) + len(self._slot_of) == self.max_requests, "a slot was lost"
        assert len(set(self._slot_of.values())) == len(self._slot_of), "a slot is held twice"
