"""The cache manager: no page is lost, held twice or freed twice, under random orders
of requests; windows give pages back; slots are reused."""

from __future__ import annotations

import random

import pytest

from mlx_omnia_b200.cache import CacheError, CacheManager, PagePool
from mlx_omnia_b200.parts.base import KVSpec, StateSpec
from mlx_omnia_b200.parts.model import CacheNeed

FULL, WINDOW = KVSpec.keys_and_values(2, 16, None), KVSpec.keys_and_values(2, 16, 10)


def manager(pages=24, page_size=4, max_requests=4):
    needs = [CacheNeed(WINDOW, None, None), CacheNeed(FULL, StateSpec((3,)), None), CacheNeed(WINDOW, None, None),
             CacheNeed(None, None, 1)]
    return CacheManager(needs, page_size=page_size, pages_per_group=pages, max_requests=max_requests, allocate=False)


def test_page_pool_refuses_double_free_and_reuses_last_freed():
    pool = PagePool(3)
    a, b = pool.take(), pool.take()
    pool.give(a)
    with pytest.raises(CacheError, match="twice"):
        pool.give(a)
    with pytest.raises(CacheError, match="not in a pool"):
        pool.give(7)
    assert pool.take() == a and pool.free == 1 and pool.held() == sorted([a, b])


def test_groups_follow_needs():
    m = manager()
    assert [g.spec for g in m.groups] == [WINDOW, FULL]
    assert m.groups[0].entries == [0, 2] and m.groups[1].entries == [1]
    assert m.group_of_entry[3] == m.group_of_entry[1]  # entry 3 reads entry 1's pages


def test_grow_is_all_or_nothing():
    m = manager(pages=3)
    r = m.open("r")
    m.grow(r, 9)
    assert [len(t) for t in r.tables] == [3, 3]
    with pytest.raises(CacheError, match="needs 1 pages, 0 free"):
        m.grow(r, 4)
    assert r.tokens == 9 and [len(t) for t in r.tables] == [3, 3]
    m.grow(r, 3)  # fills the last page, needs no new one
    m.check()


def test_window_release_arithmetic():
    m = manager(pages=32)
    r = m.open("r")
    m.grow(r, 30)
    # window 10: the next query (position 30) reads keys >= 21; pages 0..4 (positions 0..19) are dead.
    assert m.release_behind_window(r) == 5
    assert r.tables[0] == [-1] * 5 + r.tables[0][5:] and min(r.tables[1]) >= 0
    assert m.release_behind_window(r) == 0
    with pytest.raises(CacheError, match="given back"):
        m.slot_of(r, 0, 3)
    assert m.slot_of(r, 0, 21) == r.tables[0][5] * 4 + 1
    m.check()
    m.close("r")
    assert m.groups[0].pool.free == 32 and m.groups[1].pool.free == 32 and m.slots.free == 4


def test_unknown_and_duplicate_requests():
    m = manager()
    m.open("a")
    with pytest.raises(CacheError, match="already open"):
        m.open("a")
    with pytest.raises(CacheError, match="not open"):
        m.close("b")
    for name in "bcd":
        m.open(name)
    with pytest.raises(CacheError, match="slot"):
        m.open("e")


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = manager(pages=20, page_size=4, max_requests=4)
    live, counter, slots_seen = {}, 0, set()
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            name = f"r{counter}"
            counter += 1
            live[name] = m.open(name)
            slots_seen.add(live[name].slot)
            assert len({r.slot for r in live.values()}) == len(live)
        elif action < 0.85 and live:
            request = rng.choice(list(live.values()))
            count = rng.choice([1, 1, 1, 2, 5, 9, 17])
            if m.can_grow(request, count):
                before = request.tokens
                m.grow(request, count)
                assert request.tokens == before + count
                m.release_behind_window(request)
            else:
                with pytest.raises(CacheError):
                    m.grow(request, count)
        elif live:
            name = rng.choice(list(live))
            m.close(name)
            del live[name]
        m.check()
        for request in live.values():  # every position a later token may read still has a page
            for g, group in enumerate(m.groups):
                first = 0 if group.spec.window is None else max(0, request.tokens - group.spec.window + 1)
                assert all(request.tables[g][p // 4] >= 0 for p in range(first, request.tokens))
    for name in list(live):
        m.close(name)
    m.check()
    assert all(g.pool.free == g.pool.count for g in m.groups) and m.slots.free == 4 and slots_seen <= {0, 1, 2, 3}


def test_rows_of_any_shape_and_a_stride_size_their_own_pages():
    """A group's pages are made from what its entries say they keep per position: two equal rows
    (keys and values), one latent row, rows of unequal width, or a row for every fourth position."""
    import torch

    latent = KVSpec(((1, 12),))
    uneven = KVSpec(((2, 16), (2, 8)), window=None)
    sparse = KVSpec(((1, 6),), stride=4)
    needs = [CacheNeed(FULL, None, None), CacheNeed(latent, None, None), CacheNeed(uneven, None, None),
             CacheNeed(sparse, None, None)]
    m = CacheManager(needs, page_size=4, pages_per_group=10, max_requests=2, dtype=torch.float32, device="cpu")
    assert [tuple(g.pages.shape) for g in m.groups] == [(1, 10, 2, 2, 4, 16), (1, 10, 1, 1, 4, 12),
                                                       (1, 10, 4 * (2 * 16 + 2 * 8)), (1, 10, 1, 1, 4, 6)]
    assert CacheManager.bytes_per_token(needs, 2) == 2 * (64 + 12 + 48 + 2)  # the sparse row: 6 / 4, rounded up
    assert m.capacity_tokens() == 40
    r = m.open("r")
    assert m.pages_needed(r, 17) == [5, 5, 5, 2]  # 17 positions: five pages of four rows; 5 sparse rows: two
    m.grow(r, 17)
    assert [len(t) for t in r.tables] == [5, 5, 5, 2]
    assert m.pages_needed(r, 3) == [0, 0, 0, 0] and m.pages_needed(r, 16) == [4, 4, 4, 1]
    assert m.slot_of(r, 3, 13) == r.tables[3][0] * 4 + 3 and m.slot_of(r, 3, 16) == r.tables[3][1] * 4
    m.check()
    m.close("r")
    assert all(g.pool.free == 10 for g in m.groups)
    with pytest.raises(ValueError, match="positive"):
        KVSpec(())
