"""A pool of fixed-size cache pages: a LIFO free list with reference counts.

Pages are plain integers; what a page holds is the business of the group that owns the pool. The
reference's `BlockPool` is the same idea (crates/specrt/src/sched.rs:18-96): freed pages go back on
the stack and are handed out again first, so a short-lived request's pages are reused at once.
"""
from __future__ import annotations


class PagePoolError(RuntimeError):
    """A page was freed twice, or a page that was never handed out was freed or shared."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._refs = [0] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int | None:
        """One page with reference count 1, or None when the pool is empty."""
        if not self._free:
            return None
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def share(self, page: int) -> None:
        """Another holder of a page that is already held."""
        self._check_held(page, "shared")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        """Drop one reference; the page returns to the free list when nobody holds it."""
        self._check_held(page, "freed")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def _check_held(self, page: int, verb: str) -> None:
        if not 0 <= page < self.num_pages:
            raise PagePoolError(f"page {page} is outside the pool of {self.num_pages} pages")
        if self._refs[page] <= 0:
            raise PagePoolError(f"page {page} is {verb} but nobody holds it")

    def check(self) -> None:
        """Invariant: every page is either free (once, count 0) or held (count > 0), never both."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PagePoolError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._refs[p] > 0):
                raise PagePoolError(f"page {p} has reference count {self._refs[p]} but is {'on' if p in free else 'not on'} the free list")
