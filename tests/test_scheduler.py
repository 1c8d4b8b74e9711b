"""The scheduler's decisions, driven by a fake step that needs no GPU."""

import random

import pytest
import torch

from inf_engine_b200.cache import CacheManager, CacheRequirement
from inf_engine_b200.engine.scheduler import Request, Scheduler


def make(n_pages=8, page_size=4, max_requests=4, max_positions=256, **kw):
    cache = CacheManager([CacheRequirement(kind="kv", n_kv_heads=1, head_dim=16, dtype=torch.float32)],
                         page_size, n_pages, max_requests)
    return cache, Scheduler(cache, max_positions, **kw)


def run_step(cache, sched, token_of=lambda req: 7):
    """What the engine does around the model: reserve happened in plan(); advance, sample, commit."""
    plan = sched.plan()
    assert plan.n_tokens <= sched.max_tokens_per_step
    seen = set()
    for e in plan.entries:
        assert e.request.req_id not in seen
        seen.add(e.request.req_id)
        base = cache.lengths[e.request.req_id]
        assert e.tokens == e.request.tokens[base:base + len(e.tokens)]
        assert e.wants_logits == (base + len(e.tokens) == len(e.request.tokens))
        cache.advance(e.request.req_id, base + len(e.tokens))
    sampled = {e.request.req_id: token_of(e.request) for e in plan.entries if e.wants_logits}
    done = sched.commit(plan, sampled)
    cache.check()
    return plan, done


def test_prompt_is_cut_into_portions_under_the_budget():
    cache, s = make(n_pages=16, max_tokens_per_step=8, chunk=5)
    r = Request(0, list(range(13)), max_new_tokens=2)
    assert s.submit(r)
    sizes = []
    while s.has_work:
        plan, _ = run_step(cache, s)
        sizes.append([len(e.tokens) for e in plan.entries])
    assert sizes == [[5], [5], [3], [1]]
    assert r.generated == [7, 7] and cache.n_free_pages() == 16


def test_decodes_ride_with_prompt_portions_and_go_first():
    cache, s = make(n_pages=32, max_tokens_per_step=6)
    a, b = Request(0, [1, 2, 3], 4), Request(1, list(range(10)), 2)
    s.submit(a)
    run_step(cache, s)                      # a prefilled, one token generated
    s.submit(b)
    plan, _ = run_step(cache, s)
    assert [(e.request.req_id, len(e.tokens)) for e in plan.entries] == [(0, 1), (1, 5)]
    plan, _ = run_step(cache, s)
    assert [(e.request.req_id, len(e.tokens), e.wants_logits) for e in plan.entries] == [(0, 1, True), (1, 5, True)]


def test_first_come_first_served_and_waiting_for_pages():
    cache, s = make(n_pages=4, page_size=4, max_tokens_per_step=64)
    big, small = Request(0, list(range(10)), 3), Request(1, [1, 2], 2)
    blocker = Request(2, list(range(6)), 1000 // 100)
    s.submit(blocker)
    run_step(cache, s)                       # blocker holds 2 pages
    s.submit(big)                            # needs 3 pages (10+1 tokens): has to wait
    s.submit(small)                          # would fit, but does not overtake
    plan, _ = run_step(cache, s)
    assert [e.request.req_id for e in plan.entries] == [2] and plan.admitted == []
    while blocker not in s.completed:
        run_step(cache, s)
    plan, _ = run_step(cache, s)
    assert [r.req_id for r in plan.admitted][:1] == [0]


def test_requests_that_can_never_fit_are_refused_at_submit():
    cache, s = make(n_pages=4, page_size=4, max_positions=64)
    r = Request(0, list(range(10)), 10)
    assert not s.submit(r) and "never fit" in r.error
    r = Request(1, list(range(60)), 10)
    assert not s.submit(r) and "positions" in r.error
    assert not s.submit(Request(2, [], 3))
    cache2, s2 = make(max_queue_depth=1)
    assert s2.submit(Request(0, [1], 1)) and not s2.submit(Request(1, [1], 1))


def test_when_pages_run_out_the_youngest_is_preempted_and_recomputed():
    cache, s = make(n_pages=4, page_size=4, max_tokens_per_step=64)
    old, young = Request(0, list(range(6)), 9), Request(1, list(range(5)), 9)
    s.submit(old)
    s.submit(young)
    preempted_at = None
    steps = 0
    while s.has_work:
        plan, _ = run_step(cache, s, token_of=lambda r: 100 + len(r.generated))
        steps += 1
        if plan.preempted and preempted_at is None:
            preempted_at = steps
            assert [r.req_id for r in plan.preempted] == [1]          # the youngest gives way
            assert s.queue[0] is young and 1 not in cache.slots        # back at the head, everything freed
        assert steps < 200
    assert preempted_at is not None and young.preemptions >= 1 and s.n_preemptions >= 1
    # both finished with all their tokens, in order, none sampled twice
    assert old.generated == [100 + i for i in range(9)]
    assert young.generated == [100 + i for i in range(9)]
    assert cache.n_free_pages() == 4 and cache.n_free_slots == 4


def test_eos_and_stop_check_finish_early():
    cache, s = make(n_pages=64, eos_token=9)
    a = Request(0, [1, 2], 50)
    b = Request(1, [3], 50, stop_check=lambda g: len(g) >= 3)
    s.submit(a)
    s.submit(b)
    while s.has_work:
        run_step(cache, s, token_of=lambda r: 9 if (r is a and len(r.generated) == 2) else 5)
    assert a.generated == [5, 5, 9]          # the EOS token is kept (engine/llama_paged_engine.py:204-210)
    assert b.generated == [5, 5, 5]


def test_batch_cap_and_slots():
    cache, s = make(n_pages=64, max_requests=3, max_tokens_per_step=64, max_batch=2)
    for i in range(4):
        s.submit(Request(i, [1, 2, 3], 2))
    plan, _ = run_step(cache, s)
    assert len(plan.admitted) == 2 and len(s.running) == 2
    while s.has_work:
        run_step(cache, s)
    assert sorted(r.req_id for r in s.completed) == [0, 1, 2, 3]


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_with_every_page_back(seed):
    rng = random.Random(seed)
    cache, s = make(n_pages=rng.choice([6, 10, 20]), page_size=rng.choice([2, 4]), max_requests=4,
                    max_tokens_per_step=rng.choice([3, 8, 32]), chunk=rng.choice([None, 2, 5]))
    reqs = []
    for i in range(12):
        r = Request(i, [rng.randrange(50) for _ in range(rng.randrange(1, 12))], rng.randrange(1, 8))
        if s.submit(r):
            reqs.append(r)
    assert reqs
    steps = 0
    while s.has_work:
        run_step(cache, s, token_of=lambda r: len(r.generated))
        steps += 1
        assert steps < 2000
    for r in reqs:
        assert r.generated == list(range(r.max_new_tokens))
    assert cache.n_free_pages() == cache.n_pages and cache.n_free_slots == 4


def test_steps_booked_before_their_tokens_are_read():
    """One step ahead: a step is booked with placeholders; its tokens arrive a step later.  A request that
    ends by its token is found out late, its extra entry is cancelled and the placeholder dropped."""
    from inf_engine_b200.engine.scheduler import PLACEHOLDER
    cache, s = make(n_pages=64, eos_token=9)
    a, b = Request(0, [1, 2, 3], 5), Request(1, [4, 5], 3)
    s.submit(a)
    s.submit(b)
    script = {0: [5, 9, 7, 7, 7], 1: [6, 6, 6]}       # request 0 says EOS as its second token
    pending = None
    finished = []
    steps = 0
    while s.has_work or pending:
        plan = s.plan()
        for e in plan.entries:
            base = cache.lengths[e.request.req_id]
            assert all(t >= 0 for t in e.tokens[:-1])
            cache.advance(e.request.req_id, base + len(e.tokens))
        s.book(plan)
        for e in plan.entries:
            if e.wants_logits:
                assert e.request.generated[e.slot] == PLACEHOLDER
        if pending is not None:
            toks = {e.request.req_id: script[e.request.req_id][e.slot] for e in pending.entries if e.wants_logits}
            finished += s.resolve(pending, toks, plan)
        pending = plan if plan.entries else None
        cache.check()
        steps += 1
        assert steps < 50
    assert a.generated == [5, 9]                         # nothing after the EOS, no placeholder left
    assert b.generated == [6, 6, 6]                      # ended by max_new_tokens at booking time
    assert sorted(r.req_id for r in finished) == [0, 1] and s.completed == finished
    assert cache.n_free_pages() == 64 and cache.n_free_slots == 4


@pytest.mark.parametrize("seed", range(6))
def test_page_reservations_that_fail_out_of_the_blue_are_survived(seed):
    """Failure injection on the host: ``reserve`` says no (and takes nothing) at random calls, as if the pool had just
    run dry.  The scheduler never raises: a portion waits or shrinks, a decoding request preempts the youngest; every
    request still gets exactly its tokens, and every page and slot is back at the end."""
    rng = random.Random(100 + seed)
    cache, s = make(n_pages=rng.choice([8, 16]), page_size=rng.choice([2, 4]), max_requests=4,
                    max_tokens_per_step=rng.choice([4, 16]), chunk=rng.choice([None, 3]))
    true_reserve = cache.reserve
    calls = {"n": 0, "refused": 0}

    def flaky_reserve(rid, new_length):
        calls["n"] += 1
        if rng.random() < 0.25:
            calls["refused"] += 1
            return False
        return true_reserve(rid, new_length)

    cache.reserve = flaky_reserve
    reqs = []
    for i in range(10):
        r = Request(i, [rng.randrange(50) for _ in range(rng.randrange(1, 10))], rng.randrange(1, 6))
        if s.submit(r):
            reqs.append(r)
    assert reqs
    steps = 0
    while s.has_work:
        run_step(cache, s, token_of=lambda r: len(r.generated))
        steps += 1
        assert steps < 5000
    assert calls["refused"] > 0
    for r in reqs:
        assert r.generated == list(range(r.max_new_tokens)) and r.error is None
    assert cache.n_free_pages() == cache.n_pages and cache.n_free_slots == 4
