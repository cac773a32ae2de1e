"""The scheduler's decisions, with no model at all: what a step holds under a token
budget, who is admitted, what happens when pages run out, and how requests end."""

from __future__ import annotations

import random

import pytest

from mlx_omnia_b200.cache import CacheManager
from mlx_omnia_b200.engine.scheduler import Request, Scheduler
from mlx_omnia_b200.parts.base import KVSpec
from mlx_omnia_b200.parts.model import CacheNeed


def make(pages=16, page_size=4, max_requests=4, budget=16, window=None):
    needs = [CacheNeed(KVSpec.keys_and_values(1, 8, None), None, None)]
    if window:
        needs.append(CacheNeed(KVSpec.keys_and_values(1, 8, window), None, None))
    cache = CacheManager(needs, page_size=page_size, pages_per_group=pages, max_requests=max_requests, allocate=False)
    return Scheduler(cache, max_tokens_per_step=budget), cache


def run_step(scheduler, cache, next_token=lambda r: 100 + len(r.generated)):
    """What the generator does around a plan, minus the model."""
    plan = scheduler.plan()
    for e in plan.entries:
        cache.grow(e.request.cache, e.count)
        e.request.cache.fresh = False
        cache.release_behind_window(e.request.cache)
    outputs = scheduler.commit(plan, {e.request.request_id: next_token(e.request) for e in plan.entries if e.samples})
    cache.check()
    return plan, outputs


def shape(plan):
    return [(e.request.request_id, e.start, e.count, e.samples) for e in plan.entries]


def test_prompts_are_cut_under_the_budget_and_decode_goes_first():
    scheduler, cache = make(pages=32, budget=16)
    scheduler.add(Request("a", list(range(10)), 3))
    scheduler.add(Request("b", list(range(30)), 2))
    plan, _ = run_step(scheduler, cache)
    assert shape(plan) == [("a", 0, 10, True), ("b", 0, 6, False)]
    plan, _ = run_step(scheduler, cache)
    assert shape(plan) == [("a", 10, 1, True), ("b", 6, 15, False)]  # the decode token first, then the portion
    plan, outputs = run_step(scheduler, cache)
    assert shape(plan) == [("a", 11, 1, True), ("b", 21, 9, True)]
    assert [(o.request.request_id, o.token, o.finished) for o in outputs] == [("a", 102, True), ("b", 100, False)]
    assert "a" not in cache.requests  # finished: everything given back
    plan, outputs = run_step(scheduler, cache)
    assert shape(plan) == [("b", 30, 1, True)] and outputs[0].finished and scheduler.idle
    assert cache.groups[0].pool.free == 32 and cache.slots.free == 4


def test_admission_is_first_come_first_served_and_bounded():
    scheduler, cache = make(pages=64, max_requests=2, budget=64)
    for name in "abc":
        scheduler.add(Request(name, [1, 2, 3], 2))
    plan, _ = run_step(scheduler, cache)
    assert [e.request.request_id for e in plan.entries] == ["a", "b"]  # only two slots
    plan, _ = run_step(scheduler, cache)
    assert [e.request.request_id for e in plan.entries] == ["a", "b"]
    plan, _ = run_step(scheduler, cache)   # a and b ended in the previous step
    assert shape(plan) == [("c", 0, 3, True)]


def test_a_portion_shrinks_to_the_free_pages():
    scheduler, cache = make(pages=4, budget=64)
    scheduler.add(Request("a", list(range(6)), 4))
    scheduler.add(Request("b", list(range(9)), 1))
    plan, _ = run_step(scheduler, cache)
    assert shape(plan) == [("a", 0, 6, True), ("b", 0, 8, False)]  # two pages each; b's prompt is cut to them
    plan, _ = run_step(scheduler, cache)
    # a decodes into its half-empty page; b has no page to go on and waits.
    assert shape(plan) == [("a", 6, 1, True)] and not plan.preempted


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    scheduler, cache = make(pages=6, budget=64)
    scheduler.add(Request("old", list(range(8)), 8))
    scheduler.add(Request("new", list(range(7)), 8))
    plan, _ = run_step(scheduler, cache)
    assert shape(plan) == [("old", 0, 8, True), ("new", 0, 7, True)]     # 2 + 2 pages of 6
    plan, _ = run_step(scheduler, cache)
    assert shape(plan) == [("old", 8, 1, True), ("new", 7, 1, True)]     # old takes a third page
    for _ in range(3):
        plan, _ = run_step(scheduler, cache)                             # new takes the last page; both fill up
        assert not plan.preempted
    new = next(r for r in scheduler.running if r.request_id == "new")
    assert new.computed == 11 and len(new.generated) == 5
    plan, _ = run_step(scheduler, cache)
    # old needs a fourth page, none is free: the newest request gives everything back and waits.
    assert [r.request_id for r in plan.preempted] == ["new"]
    assert shape(plan) == [("old", 12, 1, True)]
    assert new.status == "waiting" and new.computed == 0 and new.cache is None and new.preemptions == 1
    assert scheduler.waiting[0] is new and len(new.generated) == 5       # what it generated is kept
    while scheduler.running:
        plan, _ = run_step(scheduler, cache)
        if any(e.request is new for e in plan.entries):
            break
    # Re-admitted: prompt and generated tokens are recomputed as one prompt, then it samples again.
    entry = next(e for e in plan.entries if e.request is new)
    assert (entry.start, entry.samples) == (0, entry.count == 12)
    while not scheduler.idle:
        run_step(scheduler, cache)
    assert len(new.generated) == 8 and new.finish_reason == "length"
    assert cache.groups[0].pool.free == 6


def test_the_only_request_is_never_starved_and_long_prompts_are_refused():
    scheduler, cache = make(pages=4, budget=64)
    with pytest.raises(ValueError, match="does not fit"):
        scheduler.add(Request("big", list(range(16)), 1))
    request = Request("fits", list(range(10)), 100)
    scheduler.add(request)
    assert request.max_tokens == 6  # cut to what the pool can hold
    while not scheduler.idle:
        plan, _ = run_step(scheduler, cache)
        assert plan.entries and not plan.preempted
    assert len(request.generated) == 6


def test_stop_tokens_end_without_being_emitted_and_abort_frees():
    scheduler, cache = make(pages=16)
    a = Request("a", [1, 2, 3], 10, stop=frozenset({101}))
    b = Request("b", [1, 2, 3, 4, 5], 10)
    scheduler.add(a)
    scheduler.add(b)
    _, outputs = run_step(scheduler, cache)
    assert [o.token for o in outputs] == [100, 100]
    _, outputs = run_step(scheduler, cache)
    assert (outputs[0].token, outputs[0].finished, a.finish_reason, a.generated) == (None, True, "stop", [100])
    assert scheduler.abort("b") is b and b.finish_reason == "abort" and scheduler.idle
    assert cache.groups[0].pool.free == 16 and not cache.requests
    c = Request("c", [1], 0)
    scheduler.add(c)
    _, outputs = run_step(scheduler, cache)
    assert outputs[0].finished and c.generated == [] and c.finish_reason == "length"


@pytest.mark.parametrize("seed", range(6))
def test_random_load_always_drains(seed):
    """Whatever arrives, every request finishes with all its tokens, the budget holds in
    every step, and all pages come back (windowed group included)."""
    rng = random.Random(seed)
    scheduler, cache = make(pages=12, page_size=4, max_requests=3, budget=13, window=6)
    requests = [Request(f"r{i}", [rng.randrange(50) for _ in range(rng.randrange(1, 30))], rng.randrange(0, 12))
                for i in range(14)]
    pending = list(requests)
    steps = 0
    while pending or not scheduler.idle:
        for _ in range(rng.randrange(0, 3)):
            if pending:
                scheduler.add(pending.pop(0))
        plan, _ = run_step(scheduler, cache)
        assert plan.num_tokens <= 13
        assert len({e.request.request_id for e in plan.entries}) == len(plan.entries)
        steps += 1
        assert steps < 3000
    assert all(r.status == "finished" and len(r.generated) == r.max_tokens for r in requests)
    assert all(g.pool.free == g.pool.count for g in cache.groups) and cache.slots.free == 3
