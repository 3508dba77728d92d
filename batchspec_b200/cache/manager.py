"""Cache manager: pages of keys and values with a block table per request, one
pool per group of layers with the same needs, and slots of fixed-size state.

The reference gives every batch slot a static range of page ids and never shares
pages between slots (batchspec/backends/utils/paging.py:196,232;
backends/base/page_table.py:55-137), doing the arithmetic with device tensors.
Here all bookkeeping is on the host: a pool is a LIFO free list shared by all
requests, a request holds ceil(len / page_size) table entries per group (none when
empty), finished requests' pages go back to the list and are handed out again, and
a windowed group also gives back pages that the window has passed (their table
entries become -1; no kernel reads them).

The pool is zeroed once when it is made and never again: what a kernel loads past a request's length is
masked, it only has to be finite.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheSpec, StateSpec


class OutOfPages(RuntimeError):
    """A reservation needs more pages than a pool has free."""


class PagePool:
    """Free list of page ids 0..num_pages-1.  ``allocate`` pops, ``free`` pushes;
    both check that no page is handed out twice or returned twice.  ``reserved``
    extra ids (num_pages .. num_pages+reserved-1) exist in the page tensor but are
    never handed out: the engine uses one as a scratch page for the padding rows of
    captured decode steps."""

    def __init__(self, num_pages: int, reserved: int = 0):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self.reserved = int(reserved)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._held = [False] * self.num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} of {self.num_pages} are free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            assert not self._held[p], f"page {p} handed out twice"
            self._held[p] = True
        self.high_water = max(self.high_water, self.num_held)
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise RuntimeError(f"page {p} freed but not held")
            self._held[p] = False
            self._free.append(p)


class StateSlots:
    """Ids 0..n-1 for per-request state of fixed size.  ``reserved`` extra ids (n ..) exist in the state tensors
    but are never handed out: the padding rows of captured decode steps read and write the first of them."""

    def __init__(self, n: int, reserved: int = 0):
        self.n = int(n)
        self.reserved = int(reserved)
        self._free = list(range(self.n - 1, -1, -1))
        self._held = [False] * self.n

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.n} request slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give(self, s: int) -> None:
        if not (0 <= s < self.n) or not self._held[s]:
            raise RuntimeError(f"slot {s} returned but not held")
        self._held[s] = False
        self._free.append(s)


@dataclass
class CacheGroup:
    """Layers whose mixers asked for the same thing share a pool and block tables."""
    spec: CacheSpec
    page_size: int
    pool: PagePool
    runs: List[int] = field(default_factory=list)        # indices into the model's order
    pages: Optional[torch.Tensor] = None       # [len(runs), num_pages, spec.tensors, page_size * entry_elems]

    @property
    def entry_elems(self) -> int:
        n = 1
        for s in self.spec.entry_shape:
            n *= s
        return n


@dataclass
class RequestCache:
    req_id: object
    slot: int
    length: int = 0
    tables: List[List[int]] = field(default_factory=list)   # per group: page id per logical page, -1 once released
    serial: int = 0     # which admission this is: a request that is released and admitted again gets a new one


class CacheManager:
    """Built from the model's per-run needs (``DecoderModel.cache_needs()``).

    ``page_size`` is the default tokens-per-page; a mixer's ``CacheSpec.page_size`` overrides it for its group.
    ``num_pages`` is the size of every group's pool in pages of the default size (a group with pages of its own
    size gets as many as hold the same number of tokens), or a list with one count per group.
    ``allocate=False`` keeps the bookkeeping only (tests, planning)."""

    def __init__(self, needs, page_size: int, num_pages, max_requests: int, dtype: torch.dtype, device,
                 allocate: bool = True, scratch_page: bool = False):
        from ..models.decoder import LayerCache
        self.page_size = int(page_size)
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        self.max_requests = int(max_requests)
        self.dtype, self.device = dtype, device
        self.groups: List[CacheGroup] = []
        self.slots = StateSlots(self.max_requests, reserved=int(scratch_page))
        self.requests: Dict[object, RequestCache] = {}
        key_to_group: Dict[Tuple, int] = {}
        run_group: Dict[int, Tuple[int, int]] = {}           # run -> (group, index in group)
        for e, need in enumerate(needs):
            if need.cache is None or need.cache_from is not None:
                continue
            c = need.cache
            if c.tensors < 1 or (c.page_size is not None and c.page_size <= 0):
                raise ValueError(f"run {e}: a cache entry has at least one tensor and a positive page size, got {c}")
            group_page = int(c.page_size or self.page_size)
            key = (c.policy, c.window, tuple(c.entry_shape), c.tensors, group_page)
            if key not in key_to_group:
                key_to_group[key] = len(self.groups)
                n = num_pages[len(self.groups)] if isinstance(num_pages, (list, tuple)) else num_pages
                if not isinstance(num_pages, (list, tuple)) and group_page != self.page_size:
                    n = -(-n * self.page_size // group_page)         # the same number of tokens in pages of its own size
                self.groups.append(CacheGroup(c, group_page, PagePool(n, reserved=int(scratch_page))))
            g = key_to_group[key]
            run_group[e] = (g, len(self.groups[g].runs))
            self.groups[g].runs.append(e)
        if allocate:
            for grp in self.groups:
                # zeroed once: kernels may load (and mask) rows of a page that no token has been written to yet,
                # and those must not hold NaN or infinity
                grp.pages = torch.zeros((len(grp.runs), grp.pool.num_pages + grp.pool.reserved, grp.spec.tensors,
                                         grp.page_size * grp.entry_elems),
                                        dtype=dtype, device=device)
        self.state_tensors: List[Optional[torch.Tensor]] = []
        self.layer_caches: List[Optional[LayerCache]] = []
        for e, need in enumerate(needs):
            state = None
            if need.state is not None and allocate:
                state = torch.zeros((self.max_requests + self.slots.reserved, *need.state.shape),
                                    dtype=need.state.dtype, device=device)
            self.state_tensors.append(state)
            owner_run = e if need.cache_from is None else need.cache_from
            if needs[owner_run].cache is None:
                kv, g = None, -1
            else:
                g, idx = run_group[owner_run]
                kv = self.groups[g].pages[idx] if allocate else None
            if kv is None and state is None and need.cache is None and need.state is None:
                self.layer_caches.append(None)
            else:
                self.layer_caches.append(LayerCache(kv=kv, group=g, state=state, owner=need.cache_from is None))

    def page_bytes(self) -> int:
        """Bytes of all pools' page tensors (whether or not they were allocated)."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.runs) * (g.pool.num_pages + g.pool.reserved) * g.spec.tensors * g.page_size * g.entry_elems * item
                   for g in self.groups)

    def scratch_pages(self) -> Optional[List[int]]:
        """Per group, the id of the page that no request ever holds (None if the
        manager was made without one)."""
        if not all(g.pool.reserved for g in self.groups):
            return None
        return [g.pool.num_pages for g in self.groups]

    def scratch_slot(self) -> Optional[int]:
        """The state slot that no request ever holds (None if the manager was made without one)."""
        return self.slots.n if self.slots.reserved else None

    # -- requests ---------------------------------------------------------------
    def admit(self, req_id) -> RequestCache:
        if req_id in self.requests:
            raise KeyError(f"request {req_id!r} is already live")
        slot = self.slots.take()
        for st in self.state_tensors:
            if st is not None:
                st[slot].zero_()
        self._admissions = getattr(self, "_admissions", 0) + 1
        rc = RequestCache(req_id, slot, 0, [[] for _ in self.groups], self._admissions)
        self.requests[req_id] = rc
        return rc

    def is_live(self, req_id) -> bool:
        return req_id in self.requests

    def length(self, req_id) -> int:
        return self.requests[req_id].length

    def pages_needed(self, length: int, n_new: int) -> List[int]:
        """Per group, the table entries a request of ``length`` tokens lacks for ``n_new`` more."""
        return [-(-(length + n_new) // g.page_size) - (-(-length // g.page_size)) for g in self.groups]

    def peak_pages(self, total_len: int, portion: int) -> List[int]:
        """Per group, the most pages one request of ``total_len`` tokens holds at any time when it is fed in
        portions of at most ``portion`` tokens: all of them in a group that keeps every key; in a window's group
        the pages from the oldest key a query still reads to the end of the portion being written (the pages the
        window has passed were given back at the commit before)."""
        out = []
        for g in self.groups:
            ps = g.page_size
            n = -(-total_len // ps)
            if g.spec.policy == "window":
                n = min(n, (g.spec.window - 1 + max(1, portion) + ps - 1) // ps + 1)
            out.append(n)
        return out

    def pages_missing(self, req_id, n_new: int) -> List[int]:
        """Per group, the pages a live request still has to get before it can take n_new more tokens (pages it
        already holds beyond its length, from a reservation that was never committed, count as held)."""
        rc = self.requests[req_id]
        return [max(0, -(-(rc.length + n_new) // g.page_size) - len(t)) for g, t in zip(self.groups, rc.tables)]

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def room_for(self, length: int, free: Sequence[int]) -> int:
        """How many more tokens a request of ``length`` tokens (holding exactly the pages of that length) can
        take with at most ``free[g]`` new pages of each group."""
        return min((f * g.page_size + (-length) % g.page_size for g, f in zip(self.groups, free)), default=1 << 60)

    def can_reserve(self, demands: Sequence[Tuple[int, int]]) -> bool:
        """demands: (current length, new tokens) per request; True if every pool
        can serve all of them together."""
        need = [0] * len(self.groups)
        for l, n in demands:
            need = [a + b for a, b in zip(need, self.pages_needed(l, n))]
        return all(n <= g.pool.num_free for n, g in zip(need, self.groups))

    def reserve(self, req_id, n_new: int) -> None:
        """Make table entries for positions length .. length+n_new-1 in every group;
        all or nothing (raises OutOfPages and leaves the request as it was)."""
        rc = self.requests[req_id]
        need = self.pages_missing(req_id, n_new)        # reserving twice for the same step is harmless
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {req_id!r} needs {n} pages, a pool has {g.pool.num_free} free")
        for n, g, table in zip(need, self.groups, rc.tables):
            if n:
                table.extend(g.pool.allocate(n))

    def commit(self, req_id, n_new: int) -> None:
        """The step wrote n_new tokens: grow the length and give back pages that a
        window has passed (every later query reads keys >= length - window + 1)."""
        rc = self.requests[req_id]
        rc.length += n_new
        for g, table in zip(self.groups, rc.tables):
            assert len(table) == -(-rc.length // g.page_size), "block table out of step"
            if g.spec.policy != "window":
                continue
            first_needed = max(0, rc.length - g.spec.window + 1)
            dead = first_needed // g.page_size             # pages wholly before first_needed
            gone = [p for p in table[:dead] if p >= 0]
            if gone:
                g.pool.free(gone)
                for i in range(dead):
                    table[i] = -1

    def release(self, req_id) -> None:
        rc = self.requests.pop(req_id)
        for g, table in zip(self.groups, rc.tables):
            g.pool.free([p for p in table if p >= 0])
        self.slots.give(rc.slot)

    def release_all(self) -> None:
        for rid in list(self.requests):
            self.release(rid)

    # -- inspection -------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, none held twice: free + held-by-requests == pool."""
        for gi, g in enumerate(self.groups):
            held = [p for rc in self.requests.values() for p in rc.tables[gi] if p >= 0]
            assert len(held) == len(set(held)), "a page is in two block tables"
            assert len(held) == g.pool.num_held, f"group {gi}: {g.pool.num_held} pages out, {len(held)} in tables"
            assert set(held).isdisjoint(g.pool._free), "a held page is on the free list"
            assert len(set(g.pool._free)) == len(g.pool._free), "a page is on the free list twice"
        assert len(self.requests) == self.slots.n - self.slots.num_free
