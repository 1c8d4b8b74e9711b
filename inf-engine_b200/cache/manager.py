"""The cache manager: pages of keys and values with a block table per request,
and slots of fixed-size state per request.

What each run of a layer needs is declared by its mixer as a
``CacheRequirement``.  Runs with the same needs (kind, heads, head size, window,
dtype) form a *group*; a group has a page pool and storage of its own, because a
group that keeps a window of keys gives pages back while another keeps all of
them.  The reference has one pool for all layers and frees only when a request
ends (engine/paged_cache.py:119-159); it has no window, no per-request state.

Life of a request:  ``open`` (takes a state slot, which is zeroed) ->
``reserve(new_length)`` before each step (takes pages; ``False`` and nothing
taken when a pool is short) -> ``advance(new_length)`` after the step (releases
pages a window has passed) -> ``close`` (everything back).

The host side (this file) is plain Python and runs without a GPU; ``allocate_storage``
makes the device tensors.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .pages import PageAccountingError, PagePool


@dataclass(frozen=True)
class CacheRequirement:
    """What one run of a layer keeps between steps.

    kind "kv": pages of keys and values, ``n_kv_heads`` x ``head_dim`` per token,
    all of them (``window`` None) or the last ``window``.
    kind "state": one tensor of ``state_shape``/``state_dtype`` per request.
    kind "none": nothing.
    """

    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None
    dtype: torch.dtype | None = None
    state_shape: tuple[int, ...] = ()
    state_dtype: torch.dtype | None = None

    def group_key(self):
        if self.kind == "kv":
            return ("kv", self.n_kv_heads, self.head_dim, self.window, self.dtype)
        if self.kind == "state":
            return ("state", self.state_shape, self.state_dtype)
        return ("none",)


@dataclass
class KVGroup:
    """Runs that share page geometry and retention; one pool, one block table per request."""

    index: int
    n_kv_heads: int
    head_dim: int
    window: int | None
    dtype: torch.dtype
    entries: list[int]                       # schedule entries (runs) stored in this group, in order
    pool: PagePool
    k: torch.Tensor | None = None            # [len(entries), n_pages, n_kv_heads, page_size, head_dim]
    v: torch.Tensor | None = None
    tables: dict = field(default_factory=dict)      # request id -> list of page ids, -1 where released
    first_live: dict = field(default_factory=dict)  # request id -> first logical page still held


@dataclass
class StateGroup:
    index: int
    shape: tuple[int, ...]
    dtype: torch.dtype
    entries: list[int]
    data: torch.Tensor | None = None         # [len(entries), max_requests, *shape]


@dataclass(frozen=True)
class CacheBinding:
    """Where one run of a layer finds its cache: group and row inside the group."""

    kind: str
    group: int = -1
    row: int = -1


class CacheManager:
    def __init__(self, requirements: list[CacheRequirement], page_size: int, n_pages: int,
                 max_requests: int, max_pages_per_request: int | None = None):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.n_pages = n_pages
        self.max_requests = max_requests
        self.max_pages_per_request = max_pages_per_request or n_pages
        self.kv_groups: list[KVGroup] = []
        self.state_groups: list[StateGroup] = []
        self.bindings: list[CacheBinding] = []
        keys: dict = {}
        for entry, req in enumerate(requirements):
            key = req.group_key()
            if req.kind == "kv":
                if key not in keys:
                    keys[key] = len(self.kv_groups)
                    self.kv_groups.append(KVGroup(len(self.kv_groups), req.n_kv_heads, req.head_dim, req.window,
                                                  req.dtype, [], PagePool(n_pages)))
                g = self.kv_groups[keys[key]]
                g.entries.append(entry)
                self.bindings.append(CacheBinding("kv", g.index, len(g.entries) - 1))
            elif req.kind == "state":
                if key not in keys:
                    keys[key] = len(self.state_groups)
                    self.state_groups.append(StateGroup(len(self.state_groups), tuple(req.state_shape),
                                                        req.state_dtype, []))
                g = self.state_groups[keys[key]]
                g.entries.append(entry)
                self.bindings.append(CacheBinding("state", g.index, len(g.entries) - 1))
            elif req.kind == "none":
                self.bindings.append(CacheBinding("none"))
            else:
                raise ValueError(f"unknown cache kind {req.kind!r}")
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.slots: dict = {}        # request id -> state slot
        self.lengths: dict = {}      # request id -> tokens held
        self.reserved: dict = {}     # request id -> tokens that pages are reserved for
        self.device = None
        # A debugging aid: pages that nobody holds are filled with NaN (all of them at the start, each one again when
        # it is given back), so that a kernel that reads a key or value it has no right to shows at once.
        self.poison_free_pages = False

    # ------------------------------------------------------------------ storage
    def allocate_storage(self, device) -> None:
        self.device = torch.device(device)
        for g in self.kv_groups:
            shape = (len(g.entries), self.n_pages, g.n_kv_heads, self.page_size, g.head_dim)
            fill = float("nan") if self.poison_free_pages else 0.0
            g.k = torch.full(shape, fill, dtype=g.dtype, device=self.device)
            g.v = torch.full(shape, fill, dtype=g.dtype, device=self.device)
        for g in self.state_groups:
            g.data = torch.zeros((len(g.entries), self.max_requests) + g.shape, dtype=g.dtype, device=self.device)

    def storage_bytes(self) -> int:
        n = 0
        for g in self.kv_groups:
            n += 2 * len(g.entries) * self.n_pages * g.n_kv_heads * self.page_size * g.head_dim * g.dtype.itemsize
        for g in self.state_groups:
            per = 1
            for s in g.shape:
                per *= s
            n += len(g.entries) * self.max_requests * per * g.dtype.itemsize
        return n

    # ------------------------------------------------------------------ requests
    def open(self, rid) -> int | None:
        """Take a state slot for a new request; ``None`` if every slot is in use."""
        if rid in self.slots:
            raise ValueError(f"request {rid!r} is already open")
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self.slots[rid] = slot
        self.lengths[rid] = 0
        self.reserved[rid] = 0
        for g in self.kv_groups:
            g.tables[rid] = []
            g.first_live[rid] = 0
        for g in self.state_groups:
            if g.data is not None:
                g.data[:, slot].zero_()
        return slot

    def _first_needed_page(self, g: KVGroup, length: int) -> int:
        """First logical page that a query at position >= ``length`` can still read."""
        if g.window is None:
            return 0
        first_key = max(0, length - g.window + 1)
        return first_key // self.page_size

    def pages_needed(self, rid, new_length: int) -> list[int]:
        """Pages each kv group would have to take so that ``rid`` can hold ``new_length`` tokens."""
        need = []
        n_logical = -(-new_length // self.page_size)
        for g in self.kv_groups:
            have = len(g.tables[rid]) if rid in g.tables else 0
            need.append(max(0, n_logical - have))
        return need

    def can_reserve(self, rid, new_length: int) -> bool:
        if -(-new_length // self.page_size) > self.max_pages_per_request:
            return False
        return all(n <= g.pool.n_free for n, g in zip(self.pages_needed(rid, new_length), self.kv_groups))

    def reserve(self, rid, new_length: int) -> bool:
        """Pages for tokens up to ``new_length`` in every group, all or nothing."""
        if rid not in self.slots:
            raise KeyError(f"request {rid!r} is not open")
        if not self.can_reserve(rid, new_length):
            return False
        for n, g in zip(self.pages_needed(rid, new_length), self.kv_groups):
            got = g.pool.allocate(n)
            assert got is not None
            g.tables[rid].extend(got)
        self.reserved[rid] = max(self.reserved[rid], new_length)
        return True

    def advance(self, rid, new_length: int) -> None:
        """Record that ``rid`` now holds ``new_length`` tokens; release pages behind every window."""
        if new_length > len(self._any_table(rid)) * self.page_size and self.kv_groups:
            raise PageAccountingError(f"request {rid!r} advanced to {new_length} beyond its reserved pages")
        self.lengths[rid] = new_length
        for g in self.kv_groups:
            if g.window is None:
                continue
            first = self._first_needed_page(g, new_length)
            table = g.tables[rid]
            lo = g.first_live[rid]
            if first > lo:
                self._give_back(g, [p for p in table[lo:first] if p >= 0])
                for i in range(lo, min(first, len(table))):
                    table[i] = -1
                g.first_live[rid] = first

    def _give_back(self, g: KVGroup, pages: list[int]) -> None:
        g.pool.free(pages)
        if self.poison_free_pages and pages and g.k is not None:
            idx = torch.tensor(pages, dtype=torch.long, device=g.k.device)
            g.k.index_fill_(1, idx, float("nan"))
            g.v.index_fill_(1, idx, float("nan"))

    def _any_table(self, rid):
        return self.kv_groups[0].tables[rid] if self.kv_groups else []

    def close(self, rid) -> None:
        """Give back every page and the state slot of ``rid``."""
        if rid not in self.slots:
            raise PageAccountingError(f"request {rid!r} closed twice or never opened")
        for g in self.kv_groups:
            self._give_back(g, [p for p in g.tables.pop(rid) if p >= 0])
            g.first_live.pop(rid)
        self._free_slots.append(self.slots.pop(rid))
        self.lengths.pop(rid)
        self.reserved.pop(rid)

    # ------------------------------------------------------------------ queries
    @property
    def n_open(self) -> int:
        return len(self.slots)

    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def n_free_pages(self) -> int:
        """Free pages of the tightest group (what admission has to look at)."""
        return min((g.pool.n_free for g in self.kv_groups), default=self.n_pages)

    def table(self, group: int, rid) -> list[int]:
        return self.kv_groups[group].tables[rid]

    def slot_of_token(self, group: int, rid, position: int) -> int:
        """Flat index ``page * page_size + offset`` of a token's keys and values."""
        page = self.kv_groups[group].tables[rid][position // self.page_size]
        if page < 0:
            raise PageAccountingError(f"position {position} of request {rid!r} lies on a released page")
        return page * self.page_size + position % self.page_size

    def check(self) -> None:
        """Raise unless every page is free or held by exactly one request, and every slot likewise."""
        for g in self.kv_groups:
            seen: dict[int, object] = {}
            for rid, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PageAccountingError(f"group {g.index}: page {p} held by {seen[p]!r} and {rid!r}")
                    if not g.pool.is_held(p):
                        raise PageAccountingError(f"group {g.index}: page {p} of {rid!r} is marked free")
                    seen[p] = rid
            if len(seen) != g.pool.n_held:
                raise PageAccountingError(
                    f"group {g.index}: {g.pool.n_held} pages marked held but {len(seen)} in block tables (a page is lost)")
            if len(set(g.pool._free)) != len(g.pool._free):
                raise PageAccountingError(f"group {g.index}: a page is on the free stack twice")
        used = sorted(self.slots.values())
        if len(set(used)) != len(used) or set(used) & set(self._free_slots):
            raise PageAccountingError("a state slot is held twice or both held and free")
        if len(used) + len(self._free_slots) != self.max_requests:
            raise PageAccountingError("a state slot is lost")
