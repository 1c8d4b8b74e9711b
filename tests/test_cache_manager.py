"""The cache manager without a GPU: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; state slots."""

import random

import pytest
import torch

from inf_engine_b200.cache import CacheManager, CacheRequirement, PageAccountingError, PagePool


def kv(window=None, heads=2, hd=16):
    return CacheRequirement(kind="kv", n_kv_heads=heads, head_dim=hd, window=window, dtype=torch.float32)


def test_pool_basics():
    # engine/paged_cache.py:39-70 has the same accounting with an exception in place of None
    pool = PagePool(4)
    a = pool.allocate(3)
    assert len(set(a)) == 3 and pool.n_free == 1
    assert pool.allocate(2) is None and pool.n_free == 1     # nothing taken on failure
    pool.free(a[:2])
    assert pool.n_free == 3
    with pytest.raises(PageAccountingError, match="twice"):
        pool.free(a[:1])
    with pytest.raises(PageAccountingError, match="outside"):
        pool.free([9])
    b = pool.allocate(3)
    assert set(b) & set(a[:2])                                # freed pages are used again
    assert pool.high_water == 4


def test_groups_are_formed_by_needs():
    m = CacheManager([kv(), kv(), kv(window=8), CacheRequirement(kind="none"), kv(window=8),
                      CacheRequirement(kind="state", state_shape=(4,), state_dtype=torch.float32)],
                     page_size=4, n_pages=8, max_requests=2)
    assert len(m.kv_groups) == 2 and len(m.state_groups) == 1
    assert m.kv_groups[0].entries == [0, 1] and m.kv_groups[1].entries == [2, 4]
    assert [b.kind for b in m.bindings] == ["kv", "kv", "kv", "none", "kv", "state"]
    assert (m.bindings[4].group, m.bindings[4].row) == (1, 1)


def test_reserve_advance_close_and_block_table():
    m = CacheManager([kv()], page_size=4, n_pages=6, max_requests=2)
    assert m.open("a") is not None
    assert m.reserve("a", 5) and len(m.table(0, "a")) == 2
    m.advance("a", 5)
    assert m.reserve("a", 8) and len(m.table(0, "a")) == 2       # still fits the second page
    assert m.reserve("a", 9) and len(m.table(0, "a")) == 3
    t = m.table(0, "a")
    assert m.slot_of_token(0, "a", 6) == t[1] * 4 + 2
    with pytest.raises(ValueError):
        m.open("a")
    assert m.open("b") is not None and m.open("c") is None        # two slots only
    assert not m.reserve("b", 13) and m.table(0, "b") == []       # 4 pages wanted, 3 free: nothing taken
    assert m.reserve("b", 12)
    m.check()
    m.close("a")
    assert m.n_free_pages() == 3
    with pytest.raises(PageAccountingError):
        m.close("a")
    with pytest.raises(PageAccountingError, match="beyond"):
        m.advance("b", 13)
    m.close("b")
    m.check()
    assert m.n_free_pages() == 6 and m.n_free_slots == 2


def test_window_group_gives_pages_back_as_it_moves():
    m = CacheManager([kv(), kv(window=6)], page_size=4, n_pages=16, max_requests=1)
    m.open("r")
    for length in range(1, 41):
        assert m.reserve("r", length)
        m.advance("r", length)
        m.check()
        full, win = m.kv_groups
        assert full.pool.n_held == -(-length // 4)
        # a query at position >= length reads keys >= length - 5: pages before that are gone
        first_needed = max(0, length - 6 + 1) // 4
        table = win.tables["r"]
        assert all(p == -1 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
        assert win.pool.n_held == len(table) - first_needed <= 3
    m.close("r")
    m.check()
    assert all(g.pool.n_free == 16 for g in m.kv_groups)


def test_state_slots_are_zeroed_when_taken():
    m = CacheManager([CacheRequirement(kind="state", state_shape=(3,), state_dtype=torch.float32), kv()],
                     page_size=4, n_pages=4, max_requests=2)
    m.allocate_storage("cpu")
    s = m.open("a")
    m.state_groups[0].data[0, s] += 5.0
    m.close("a")
    s2 = m.open("b")
    assert s2 == s and float(m.state_groups[0].data[0, s2].abs().sum()) == 0.0
    assert m.kv_groups[0].k.shape == (1, 4, 2, 4, 16)
    assert m.storage_bytes() == 2 * 4 * 2 * 4 * 16 * 4 + 2 * 3 * 4


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    m = CacheManager([kv(), kv(window=rng.choice([5, 9, 17]))], page_size=rng.choice([2, 4, 8]), n_pages=24,
                     max_requests=5)
    live: dict[int, int] = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and m.n_free_slots:
            assert m.open(next_id) is not None
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.choice([1, 1, 1, 2, 7, 19])
            free_before = [g.pool.n_free for g in m.kv_groups]
            if m.reserve(rid, new):
                m.advance(rid, new)
                live[rid] = new
            else:
                assert [g.pool.n_free for g in m.kv_groups] == free_before
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check()
        assert m.lengths == live
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(g.pool.n_free == 24 for g in m.kv_groups) and m.n_free_slots == 5


def test_pages_nobody_holds_can_be_filled_with_nan():
    """The debugging aid behind ``trace_run --poison-free-pages``: every page starts as NaN and is NaN again once it is
    given back, at the end of a request or when a window has passed it."""
    reqs = [CacheRequirement(kind="kv", n_kv_heads=1, head_dim=4, window=None, dtype=torch.float32),
            CacheRequirement(kind="kv", n_kv_heads=1, head_dim=4, window=8, dtype=torch.float32)]
    m = CacheManager(reqs, page_size=4, n_pages=6, max_requests=2)
    m.poison_free_pages = True
    m.allocate_storage("cpu")
    full, win = m.kv_groups
    assert torch.isnan(full.k).all() and torch.isnan(win.v).all()
    m.open("a")
    assert m.reserve("a", 10)
    for g in (full, win):
        for p in g.tables["a"]:
            g.k[:, p] = 1.0
            g.v[:, p] = 1.0
    m.advance("a", 10)                                   # a query at position 10 sees keys 3..10: nothing passed yet
    assert not torch.isnan(win.k[:, win.tables["a"][0]]).any()
    assert m.reserve("a", 16)
    m.advance("a", 16)                                   # keys 9..16: the first two pages of the window group go back
    gone = [p for p in range(6) if not win.pool.is_held(p)]
    assert len(gone) == 6 - 2 and all(torch.isnan(win.k[:, p]).all() and torch.isnan(win.v[:, p]).all() for p in gone)
    held = [p for p in full.tables["a"]]
    assert not torch.isnan(full.k[:, held[:3]]).any()    # the full group still holds every page it wrote
    m.close("a")
    assert torch.isnan(full.k).all() and torch.isnan(win.k).all()
    m.check()
