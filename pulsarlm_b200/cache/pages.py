"""Page ids of one pool: taken all-or-nothing, given back once, reused last-in first-out.

The reference's allocator hands out power-of-two blocks from regions and keeps
released lines as a prefix cache until reclaimed
(pulsarlm-core/src/engine/line_allocator.cpp:139-202). Here every page of a group
has one size and nothing is shared between requests, so a free stack is enough;
its order is deterministic, which makes page reuse in replayed traces repeatable.
"""

from __future__ import annotations


class PageError(RuntimeError):
    """A page was given back twice, or was never taken."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 0:
            raise ValueError(f"a pool cannot have {n_pages} pages")
        self.n_pages = n_pages
        # Stack: the page given back last is taken first; initially page 0 is on top.
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages
        self.high_water = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.n_pages - len(self._free)

    def take(self, count: int) -> list[int] | None:
        """`count` pages, or None (and nothing taken) when fewer are free."""
        if count < 0:
            raise ValueError("cannot take a negative number of pages")
        if count > len(self._free):
            return None
        taken = [self._free.pop() for _ in range(count)]
        for page in taken:
            self._held[page] = True
        self.high_water = max(self.high_water, self.used_count)
        return taken

    def give(self, pages) -> None:
        for page in pages:
            if not 0 <= page < self.n_pages or not self._held[page]:
                raise PageError(f"page {page} is given back but is not held")
            self._held[page] = False
            self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]
