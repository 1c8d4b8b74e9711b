"""A pool of fixed-size pages: a free stack with checks against loss and double use.

The reference's ``BlockManager`` is a Python list used as a stack whose
``allocate`` raises on exhaustion (engine/paged_cache.py:39-70).  This pool
returns ``None`` instead, so that running out is a decision of the caller, and
it refuses to free a page that is already free.
"""

from __future__ import annotations


class PageAccountingError(RuntimeError):
    """A page was freed twice, freed without being held, or is out of range."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        # pop() hands out low ids first
        self._free = list(range(n_pages - 1, -1, -1))
        self._held = [False] * n_pages
        self.high_water = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def allocate(self, n: int) -> list[int] | None:
        """``n`` pages, or ``None`` (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.high_water = max(self.high_water, self.n_held)
        return out

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages:
                raise PageAccountingError(f"page {p} is outside the pool of {self.n_pages}")
            if not self._held[p]:
                raise PageAccountingError(f"page {p} freed twice or never held")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]
