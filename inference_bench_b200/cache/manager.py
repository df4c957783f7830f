"""The cache manager: pages of keys and values with a block table per request, in groups of layers
with the same needs, and beside them slots of fixed-size per-request state.

Executions of the schedule whose mixers ask for the same `PagedKV(kv_heads, head_dim, window)` form a
group. A group has its own page pool, its own device tensor
[executions, pages, 2 (K, V), kv_heads, page_size, head_dim] and its own block table per request; a
page therefore holds `page_size` positions of every execution in the group, and one table serves
them all (block-major, like the reference: docs/specrt-scheduler.md:11, 20-22). A group with a window
gives a page back as soon as every position in it has fallen out of the window of the request's
next token; a request's end gives everything back. Mixers that ask for `FixedState(shape, dtype)`
get a tensor [slots, *shape], zeroed for a slot when a request is admitted to it
(reference: crates/specrt/src/statepool.rs:7-80, crates/specrt/src/runtime/step.rs:133-135).

The bookkeeping is host-only and runs without a device (tensors are made only when a device is given).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Hashable, Optional, Sequence

import numpy as np

from ..parts.base import FixedState, PagedKV
from .pages import PagePool


class OutOfPages(RuntimeError):
    """A request could not get the pages it needs for its next tokens."""


class CacheError(RuntimeError):
    """The cache manager was used wrongly (unknown request, request admitted twice, no free slot)."""


@dataclass
class Group:
    need: PagedKV
    entries: list[int]          # schedule entries whose keys and values live in this group's pages
    pool: PagePool
    tensor: Any = None          # device tensor, None without a device

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class _Request:
    slot: int
    length: int = 0                                   # positions whose state is in the cache
    tables: list[np.ndarray] = field(default_factory=list)   # per group: page id per page index, -1 = none


@dataclass
class StateView:
    """Fixed-size state of one execution: `tensor[slot]` belongs to the request in that slot."""
    tensor: Any


class CacheManager:
    def __init__(self, needs: Sequence[Any], page_size: int, num_pages: int, max_requests: int, max_tokens_per_request: int,
                 device=None, dtype=None, sources: Optional[Sequence[int]] = None):
        """needs[i]: PagedKV, FixedState or None for schedule entry i; sources[i]: the entry whose
        cache entry i uses (itself by default). num_pages: pages of every group's pool."""
        if page_size <= 0 or max_requests <= 0 or max_tokens_per_request <= 0:
            raise ValueError("page_size, max_requests and max_tokens_per_request must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.table_width = -(-max_tokens_per_request // page_size)
        self.max_tokens_per_request = max_tokens_per_request
        self.device, self.dtype = device, dtype
        self.sources = list(sources) if sources is not None else list(range(len(needs)))
        self.groups: list[Group] = []
        self.place: dict[int, tuple[int, int]] = {}    # schedule entry -> (group index, index inside the page)
        self.states: dict[int, StateView] = {}         # schedule entry -> fixed state
        by_need: dict[PagedKV, int] = {}
        for i, need in enumerate(needs):
            if isinstance(need, PagedKV):
                g = by_need.get(need)
                if g is None:
                    g = by_need[need] = len(self.groups)
                    self.groups.append(Group(need, [], PagePool(num_pages)))
                self.place[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, FixedState):
                self.states[i] = StateView(None)
            elif need is not None:
                raise TypeError(f"schedule entry {i} asks the cache for {need!r}, which it does not know")
        self._fixed = {i: n for i, n in enumerate(needs) if isinstance(n, FixedState)}
        if device is not None:
            import torch
            for g in self.groups:
                n = g.need
                # one page more than the pool hands out: the scratch page that padded rows of a fixed-size batch write to
                g.tensor = torch.zeros((len(g.entries), g.pool.num_pages + 1, 2, n.kv_heads, page_size, n.head_dim), dtype=dtype, device=device)
            for i, n in self._fixed.items():
                # and one scratch slot more than requests can hold
                self.states[i].tensor = torch.zeros((max_requests + 1, *n.shape), dtype=n.dtype, device=device)
        self._requests: dict[Hashable, _Request] = {}
        self._free_slots = list(range(max_requests - 1, -1, -1))

    @property
    def scratch_slot(self) -> int:
        return self.max_requests

    def scratch_page(self, group: int) -> int:
        return self.groups[group].pool.num_pages

    # ------------------------------------------------------------------ requests
    def live(self) -> list[Hashable]:
        return list(self._requests)

    def has(self, req: Hashable) -> bool:
        return req in self._requests

    def free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, req: Hashable) -> int:
        """Give the request a state slot (zeroed) and empty block tables."""
        if req in self._requests:
            raise CacheError(f"request {req!r} is already admitted")
        if not self._free_slots:
            raise CacheError(f"no free slot: {self.max_requests} requests are live")
        slot = self._free_slots.pop()
        self._requests[req] = _Request(slot, 0, [np.full(self.table_width, -1, dtype=np.int32) for _ in self.groups])
        for view in self.states.values():
            if view.tensor is not None:
                view.tensor[slot].zero_()
        return slot

    def _get(self, req: Hashable) -> _Request:
        try:
            return self._requests[req]
        except KeyError:
            raise CacheError(f"request {req!r} is not admitted") from None

    def slot(self, req: Hashable) -> int:
        return self._get(req).slot

    def length(self, req: Hashable) -> int:
        return self._get(req).length

    # ------------------------------------------------------------------ pages
    def _first_live_page(self, g: Group, length: int) -> int:
        """Pages below this index hold only positions that no token at position >= length can see."""
        if g.window is None:
            return 0
        return max(0, length - g.window + 1) // self.page_size

    def pages_missing(self, req: Optional[Hashable], new_length: int, length: int = 0) -> list[int]:
        """Per group, the pages that must be allocated before the request holds `new_length` positions.
        For a request not yet admitted pass req=None and the length it would start from."""
        out = []
        r = self._requests.get(req) if req is not None else None
        cur = r.length if r is not None else length
        for gi, g in enumerate(self.groups):
            first = self._first_live_page(g, cur)
            last = -(-new_length // self.page_size)
            if r is None:
                out.append(max(0, last - first))
            else:
                out.append(int(np.count_nonzero(r.tables[gi][first:last] < 0)))
        return out

    def can_extend(self, req: Optional[Hashable], new_length: int, length: int = 0, reserve: int = 0) -> bool:
        if new_length > self.max_tokens_per_request:
            return False
        return all(m + reserve <= g.pool.free_pages for m, g in zip(self.pages_missing(req, new_length, length), self.groups))

    def extend(self, req: Hashable, new_length: int) -> None:
        """Allocate, in every group, the pages for positions up to new_length - 1. All or nothing."""
        r = self._get(req)
        if new_length > self.max_tokens_per_request:
            raise OutOfPages(f"request {req!r} would hold {new_length} tokens, more than the limit of {self.max_tokens_per_request}")
        taken: list[tuple[int, int]] = []
        for gi, g in enumerate(self.groups):
            first = self._first_live_page(g, r.length)
            last = -(-new_length // self.page_size)
            for p in (np.nonzero(r.tables[gi][first:last] < 0)[0] + first).tolist():
                page = g.pool.allocate()
                if page is None:
                    for gj, pj in taken:
                        self.groups[gj].pool.release(int(r.tables[gj][pj]))
                        r.tables[gj][pj] = -1
                    raise OutOfPages(f"request {req!r} needs a page for positions {p * self.page_size}.. but group {gi} has none free "
                                     f"({g.pool.num_pages} pages, all in use)")
                r.tables[gi][p] = page
                taken.append((gi, p))

    def shrink_to_committed(self, req: Hashable) -> None:
        """Undo an `extend` that no `commit` followed: free the pages beyond the committed length."""
        r = self._get(req)
        keep = -(-r.length // self.page_size)
        for gi, g in enumerate(self.groups):
            row = r.tables[gi]
            for p in np.nonzero(row[keep:] >= 0)[0] + keep:
                g.pool.release(int(row[p]))
                row[p] = -1

    def commit(self, req: Hashable, new_length: int) -> None:
        """The request now holds new_length positions; windowed groups give back pages that passed."""
        r = self._get(req)
        r.length = new_length
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            first = self._first_live_page(g, new_length)
            row = r.tables[gi]
            for p in np.nonzero(row[:first] >= 0)[0]:
                g.pool.release(int(row[p]))
                row[p] = -1

    def release(self, req: Hashable) -> None:
        """The request ends: all its pages and its slot are given back."""
        r = self._get(req)
        for gi, g in enumerate(self.groups):
            for page in r.tables[gi][r.tables[gi] >= 0]:
                g.pool.release(int(page))
        self._free_slots.append(r.slot)
        del self._requests[req]

    def table(self, group: int, req: Hashable) -> np.ndarray:
        return self._get(req).tables[group]

    def used_pages(self) -> list[int]:
        return [g.pool.used_pages for g in self.groups]

    def free_pages(self) -> list[int]:
        return [g.pool.free_pages for g in self.groups]

    # ------------------------------------------------------------------ what a step hands to the parts
    def step_tables(self, reqs: Sequence[Hashable]) -> list[np.ndarray]:
        """Per group, the block tables of the step's segments, int32 [segments, table_width]."""
        return [np.stack([self._get(r).tables[gi] for r in reqs]) if reqs else np.zeros((0, self.table_width), np.int32)
                for gi in range(len(self.groups))]

    def views(self, device_tables: Sequence[Any]) -> list[Any]:
        """Per schedule entry, what its mixer gets this step: a KvLayerView on its group's tensor
        (its own place in the page, or that of the entry whose cache it reads), a StateView, or None."""
        from ..kernels.ops import KvLayerView
        out = []
        for i, src in enumerate(self.sources):
            if src in self.place:
                g, e = self.place[src]
                out.append(KvLayerView(self.groups[g].tensor, e, device_tables[g]))
            elif src in self.states:
                out.append(self.states[src])
            else:
                out.append(None)
        return out

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """No page lost, held twice or freed twice: every pool is consistent and a page's reference
        count equals the number of table entries that name it."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            counts = np.zeros(g.pool.num_pages, dtype=np.int64)
            for r in self._requests.values():
                held = r.tables[gi][r.tables[gi] >= 0]
                np.add.at(counts, held, 1)
            for p in range(g.pool.num_pages):
                if counts[p] != g.pool.refcount(p):
                    raise CacheError(f"group {gi}: page {p} is named by {counts[p]} table entries but has reference count {g.pool.refcount(p)}")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots) or len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("state slots are inconsistent: a slot is lost, held twice or both held and free")
