"""Page ids of one pool: taken all-or-nothing, given back once, reused last-in first-out.

The pool itself is C++ (pulsarlm_b200/csrc_host/host_core.cpp, class PagePool); this
is its Python face. The reference's allocator hands out power-of-two blocks from
regions and keeps released lines as a prefix cache until reclaimed
(pulsarlm-core/src/engine/line_allocator.cpp:139-202). Here every page of a group
has one size and nothing is shared between requests, so a free stack is enough;
its order is deterministic, which makes page reuse in replayed traces repeatable.
"""

from __future__ import annotations

import ctypes

from ..host import core


class PageError(RuntimeError):
    """A page was given back twice, or was never taken."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError(f"a pool cannot have {n_pages} pages")
        self._lib = core.library()
        self._pool = self._lib.plh_pool_create(n_pages)
        self.n_pages = n_pages

    def __del__(self):
        if getattr(self, "_pool", None):
            self._lib.plh_pool_destroy(self._pool)
            self._pool = None

    @property
    def free_count(self) -> int:
        return self._lib.plh_pool_stat(self._pool, 1)

    @property
    def used_count(self) -> int:
        return self._lib.plh_pool_stat(self._pool, 2)

    @property
    def high_water(self) -> int:
        return self._lib.plh_pool_stat(self._pool, 3)

    def take(self, count: int) -> list[int] | None:
        """`count` pages, or None (and nothing taken) when fewer are free."""
        if count < 0:
            raise ValueError("cannot take a negative number of pages")
        out = (ctypes.c_int32 * max(count, 1))()
        if self._lib.plh_pool_take(self._pool, count, out) < 0:
            return None
        return list(out[:count])

    def give(self, pages) -> None:
        pages = list(pages)
        array = (ctypes.c_int32 * max(len(pages), 1))(*pages)
        if self._lib.plh_pool_give(self._pool, array, len(pages)) != 0:
            raise PageError(f"a page of {pages} is given back but is not held")

    def is_held(self, page: int) -> bool:
        return bool(self._lib.plh_pool_is_held(self._pool, page))


class GroupPoolView:
    """Read-only figures of one group's pool inside a cache book."""

    def __init__(self, lib, book, group: int, n_pages: int):
        self._lib, self._book, self._group, self.n_pages = lib, book, group, n_pages

    @property
    def free_count(self) -> int:
        return self._lib.plh_cache_pool_stat(self._book, self._group, 1)

    @property
    def used_count(self) -> int:
        return self._lib.plh_cache_pool_stat(self._book, self._group, 2)

    @property
    def high_water(self) -> int:
        return self._lib.plh_cache_pool_stat(self._book, self._group, 3)

    def is_held(self, page: int) -> bool:
        return bool(self._lib.plh_cache_pool_is_held(self._book, self._group, page))
