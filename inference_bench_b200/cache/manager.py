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
Pools, block tables and slots live in the C++ core (csrc/host/cache_core.cpp); this class maps request
ids to slots, owns the device tensors and hands the parts their views.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Hashable, Optional, Sequence

import ctypes as C

import numpy as np

from ..parts.base import FixedState, PagedKV
from . import native
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


class _Request:
    """A live request as the core sees it: its slot, its committed length and, per group, its row of the block table."""
    __slots__ = ("slot", "_mgr")

    def __init__(self, slot: int, mgr: "CacheManager"):
        self.slot, self._mgr = slot, mgr

    @property
    def length(self) -> int:                          # positions whose state is in the cache
        return int(self._mgr._lib.ibh_cache_length(self._mgr._core, self.slot))

    @property
    def tables(self) -> list[np.ndarray]:             # per group: page id per page index, -1 = none (views of the core's memory)
        return [t[self.slot] for t in self._mgr._tables]


@dataclass
class StateView:
    """Fixed-size state of one execution: `tensor[slot]` belongs to the request in that slot.

    A mixer reads and writes the state of the step's segments through `gather` and `scatter`, which index with the
    device copy of the segments' slots (`ctx.seg_slot`). That is the only form that is right inside a captured decode
    step: there the host-side segments are placeholders and only the device arrays are filled in before each replay.
    Padded rows of such a step carry the scratch slot (the tensor's last row), which no request ever owns."""
    tensor: Any

    def gather(self, ctx) -> Any:
        """The state of every segment of the step, [segments, *shape] (a copy)."""
        return self.tensor.index_select(0, ctx.seg_slot.long())

    def scatter(self, ctx, values) -> None:
        """Store `values` [segments, *shape] as the new state of the step's segments."""
        self.tensor.index_copy_(0, ctx.seg_slot.long(), values.to(self.tensor.dtype))


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
                    self.groups.append(Group(need, [], None))
                self.place[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, FixedState):
                self.states[i] = StateView(None)
            elif need is not None:
                raise TypeError(f"schedule entry {i} asks the cache for {need!r}, which it does not know")
        self._fixed = {i: n for i, n in enumerate(needs) if isinstance(n, FixedState)}
        self._lib = native.load()
        windows = (C.c_int * max(1, len(self.groups)))(*[int(g.need.window or 0) for g in self.groups])
        self._core = self._lib.ibh_cache_new(len(self.groups), windows, page_size, num_pages, max_requests, max_tokens_per_request)
        if not self._core:
            raise ValueError(native.last_error())
        for gi, g in enumerate(self.groups):
            g.pool = PagePool(0, _handle=self._lib.ibh_cache_pool(self._core, gi))
        base = self._lib.ibh_cache_tables(self._core)
        whole = np.ctypeslib.as_array(base, shape=(max(1, len(self.groups)), max_requests, self.table_width)) if self.groups else np.zeros((0, max_requests, self.table_width), np.int32)
        self._tables = [whole[gi] for gi in range(len(self.groups))]     # per group: int32 [max_requests, table_width], the core's own memory
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

    def __del__(self):
        core, self._core = getattr(self, "_core", None), None
        if core:
            self._lib.ibh_cache_free(core)

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
        return int(self._lib.ibh_cache_free_slots(self._core))

    def admit(self, req: Hashable) -> int:
        """Give the request a state slot (zeroed) and empty block tables."""
        if req in self._requests:
            raise CacheError(f"request {req!r} is already admitted")
        slot = int(self._lib.ibh_cache_admit(self._core))
        if slot < 0:
            raise CacheError(f"no free slot: {self.max_requests} requests are live")
        self._requests[req] = _Request(slot, self)
        for view in self.states.values():
            if view.tensor is not None:
                view.tensor[slot].zero_()
        return slot

    def _adopt(self, req: Hashable, slot: int) -> None:
        """The scheduler's core admitted this request to `slot` itself: take note, and zero its fixed-size state."""
        if req in self._requests:
            raise CacheError(f"request {req!r} is already admitted")
        self._requests[req] = _Request(slot, self)
        for view in self.states.values():
            if view.tensor is not None:
                view.tensor[slot].zero_()

    def _forget(self, req: Hashable) -> None:
        """The scheduler's core gave back what this request held: drop it from the map."""
        self._requests.pop(req, None)

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
    def pages_missing(self, req: Optional[Hashable], new_length: int, length: int = 0) -> list[int]:
        """Per group, the pages that must be allocated before the request holds `new_length` positions.
        For a request not yet admitted pass req=None and the length it would start from."""
        r = self._requests.get(req) if req is not None else None
        out = (C.c_int * max(1, len(self.groups)))()
        self._lib.ibh_cache_pages_missing(self._core, r.slot if r is not None else -1, int(new_length), int(length), out)
        return [int(out[gi]) for gi in range(len(self.groups))]

    def can_extend(self, req: Optional[Hashable], new_length: int, length: int = 0, reserve: int = 0) -> bool:
        if new_length > self.max_tokens_per_request:
            return False
        return all(m + reserve <= g.pool.free_pages for m, g in zip(self.pages_missing(req, new_length, length), self.groups))

    def extend(self, req: Hashable, new_length: int) -> None:
        """Allocate, in every group, the pages for positions up to new_length - 1. All or nothing."""
        r = self._get(req)
        code = self._lib.ibh_cache_extend(self._core, r.slot, int(new_length))
        if code == 1:
            raise OutOfPages(f"request {req!r} {native.last_error()}")
        if code == 2:
            raise OutOfPages(f"request {req!r} would hold {new_length} tokens, more than the limit of {self.max_tokens_per_request}")
        if code:
            raise CacheError(native.last_error())

    def shrink_to_committed(self, req: Hashable) -> None:
        """Undo an `extend` that no `commit` followed: free the pages beyond the committed length."""
        if self._lib.ibh_cache_shrink_to_committed(self._core, self._get(req).slot):
            raise CacheError(native.last_error())

    def commit(self, req: Hashable, new_length: int) -> None:
        """The request now holds new_length positions; windowed groups give back pages that passed."""
        if self._lib.ibh_cache_commit(self._core, self._get(req).slot, int(new_length)):
            raise CacheError(native.last_error())

    def release(self, req: Hashable) -> None:
        """The request ends: all its pages and its slot are given back."""
        if self._lib.ibh_cache_release(self._core, self._get(req).slot):
            raise CacheError(native.last_error())
        del self._requests[req]

    def table(self, group: int, req: Hashable) -> np.ndarray:
        return self._get(req).tables[group]

    def used_pages(self) -> list[int]:
        return [g.pool.used_pages for g in self.groups]

    def free_pages(self) -> list[int]:
        return [g.pool.free_pages for g in self.groups]

    def fill_rows(self, reqs: Sequence[Hashable], positions: np.ndarray, tables: Sequence[np.ndarray]) -> list[int]:
        """For a step of single decoded tokens: write the requests' committed lengths (their next positions)
        into positions[:n] and their block tables into tables[g][:n] (int32, contiguous; typically the pinned
        input block of a captured step), in one call into the core. Returns the requests' slots."""
        n = len(reqs)
        slots = [self._get(r).slot for r in reqs]
        arr = (C.c_int * max(1, n))(*slots)
        ptrs = (C.POINTER(C.c_int) * max(1, len(tables)))(*[t.ctypes.data_as(C.POINTER(C.c_int)) for t in tables])
        if self._lib.ibh_cache_fill_rows(self._core, arr, n, positions.ctypes.data_as(C.POINTER(C.c_int)), ptrs):
            raise CacheError(native.last_error())
        return slots

    # ------------------------------------------------------------------ what a step hands to the parts
    def step_tables(self, reqs: Sequence[Hashable]) -> list[np.ndarray]:
        """Per group, the block tables of the step's segments, int32 [segments, table_width]."""
        slots = [self._get(r).slot for r in reqs]
        return [t[slots] if slots else np.zeros((0, self.table_width), np.int32) for t in self._tables]

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
        if self._lib.ibh_cache_check(self._core):
            raise CacheError(native.last_error())
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or len(slots) + self.free_slots() != self.max_requests:
            raise CacheError("state slots are inconsistent: a slot is lost, held twice or both held and free")
