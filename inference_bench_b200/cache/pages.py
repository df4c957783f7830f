"""A pool of fixed-size cache pages: a LIFO free list with reference counts.

Pages are plain integers; what a page holds is the business of the group that owns the pool. The
bookkeeping itself is C++ (csrc/host/cache_core.cpp); this class is its Python face. The reference's
`BlockPool` is the same idea (crates/specrt/src/sched.rs:18-96): freed pages go back on the stack and
are handed out again first, so a short-lived request's pages are reused at once.
"""
from __future__ import annotations

from . import native


class PagePoolError(RuntimeError):
    """A page was freed twice, or a page that was never handed out was freed or shared."""


class PagePool:
    def __init__(self, num_pages: int, _handle=None):
        """A pool of its own, or (with `_handle`) the face of a pool that a cache core owns."""
        self._lib = native.load()
        if _handle is None:
            if num_pages <= 0:
                raise ValueError(f"a page pool needs at least one page, got {num_pages}")
            self._h, self._own = self._lib.ibh_pool_new(num_pages), True
        else:
            self._h, self._own = _handle, False
        self.num_pages = int(self._lib.ibh_pool_num_pages(self._h))

    def __del__(self):
        if getattr(self, "_own", False) and self._h:
            self._lib.ibh_pool_free(self._h)
            self._h = None

    @property
    def free_pages(self) -> int:
        return int(self._lib.ibh_pool_free_pages(self._h))

    @property
    def used_pages(self) -> int:
        return self.num_pages - self.free_pages

    def allocate(self) -> int | None:
        """One page with reference count 1, or None when the pool is empty."""
        page = int(self._lib.ibh_pool_allocate(self._h))
        return None if page < 0 else page

    def share(self, page: int) -> None:
        """Another holder of a page that is already held."""
        if self._lib.ibh_pool_share(self._h, int(page)):
            raise PagePoolError(native.last_error())

    def release(self, page: int) -> None:
        """Drop one reference; the page returns to the free list when nobody holds it."""
        if self._lib.ibh_pool_release(self._h, int(page)):
            raise PagePoolError(native.last_error())

    def refcount(self, page: int) -> int:
        return int(self._lib.ibh_pool_refcount(self._h, int(page)))

    def check(self) -> None:
        """Invariant: every page is either free (once, count 0) or held (count > 0), never both."""
        if self._lib.ibh_pool_check(self._h):
            raise PagePoolError(native.last_error())
