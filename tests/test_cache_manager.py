"""The cache manager on the host: no page lost, held twice or freed twice, under random orders
of requests; windows give pages back; reservations hold."""

import random

import pytest
import torch

from mlx_one_b200.cache import (CacheCapacityError, CacheManager, CacheOwnershipError,
                                IndexPool)
from mlx_one_b200.parts.base import FixedState, PagedKeyValues

NEEDS = {0: FixedState((2, 8)), 1: PagedKeyValues(2, 16), 2: FixedState((2, 8)),
         3: PagedKeyValues(2, 16), 4: PagedKeyValues(2, 16, window=10),
         5: PagedKeyValues(1, 32)}


def manager(capacity=64, page=4, requests=4, step=1 << 30, allocate=False):
    return CacheManager(NEEDS, page_size=page, capacity_tokens=capacity, max_requests=requests,
                        dtype=torch.float32, device="cpu", max_step_tokens=step,
                        allocate=allocate)


def test_pool_hands_back_last_freed_first_and_refuses_double_free():
    pool = IndexPool(3)
    a, b = pool.take(), pool.take()
    pool.give_back(a)
    assert pool.take() == a                      # reuse as early as possible
    pool.give_back(b)
    with pytest.raises(CacheOwnershipError):
        pool.give_back(b)
    with pytest.raises(CacheOwnershipError):
        pool.give_back(17)
    pool.take(), pool.take()
    with pytest.raises(CacheCapacityError) as caught:
        pool.take()
    assert caught.value.retryable


def test_layers_with_equal_needs_share_a_group():
    cache = manager(allocate=True)
    assert len(cache.paged) == 3 and len(cache.states) == 1
    assert cache.locate(1)[:2] == cache.locate(3)[:2] == ("paged", 0)
    assert cache.locate(4)[1] != cache.locate(1)[1]          # the window has pages of its own
    # 16 pages and 4 slots for requests, and the scratch page and slot that none of them gets
    assert cache.paged[0].storage.shape == (2, 2, 16 + 1, 2, 4, 16)
    assert cache.states[0].storage.shape == (2, 4 + 1, 2, 8)
    assert cache.scratch_page == 16 and cache.scratch_slot == 4
    assert cache.paged[0].pool.count == 16 and cache.states[0].pool.count == 4


def test_grow_advance_close_and_window_release():
    cache = manager()
    cache.open("a")
    cache.grow("a", 9)
    cache.advance("a", 9)
    held = cache.get("a")
    assert [len(t) for t in held.tables] == [3, 3, 3]
    cache.grow("a", 30)
    cache.advance("a", 30)                                    # 39 tokens, window 10
    window_group = cache.locate(4)[1]
    table = held.tables[window_group]
    # the next query (position 39) reads keys 30..39: blocks 0..6 (tokens 0..27) are given back
    assert table[:7] == [-1] * 7 and all(p >= 0 for p in table[7:])
    assert held.live[window_group] == 3
    cache.check()
    cache.close("a")
    assert cache.stats().pages_free == cache.stats().pages_total
    with pytest.raises(CacheOwnershipError):
        cache.close("a")
    with pytest.raises(CacheOwnershipError):
        cache.grow("a", 1)


def test_running_out_of_pages_takes_nothing():
    cache = manager(capacity=16)
    cache.open("a")
    cache.open("b")
    cache.grow("a", 12)
    before = cache.stats()
    with pytest.raises(CacheCapacityError) as caught:
        cache.grow("b", 8)
    assert caught.value.retryable
    assert cache.stats() == before
    cache.check()


def test_reservations_hold_and_limit():
    cache = manager(capacity=32)
    assert not cache.fits_ever(33) and cache.fits_ever(32)
    with pytest.raises(CacheCapacityError) as caught:
        cache.open("big", reserve_tokens=33)
    assert not caught.value.retryable
    cache.open("a", reserve_tokens=20)
    with pytest.raises(CacheCapacityError) as caught:
        cache.open("b", reserve_tokens=16)                    # 5 + 4 pages > 8
    assert caught.value.retryable and "b" not in cache
    cache.open("c")                                           # unreserved
    cache.grow("c", 12)                                       # takes the 3 unpromised pages
    cache.advance("c", 12)
    with pytest.raises(CacheCapacityError):
        cache.grow("c", 1)                                    # the rest is promised to "a"
    cache.grow("a", 20)                                       # cannot fail
    cache.advance("a", 20)
    with pytest.raises(CacheCapacityError) as caught:
        cache.grow("a", 1)                                    # beyond its reservation
    assert not caught.value.retryable
    cache.check()
    cache.close("a")
    cache.grow("c", 4)
    cache.check()


def test_window_group_reserves_less_than_the_whole_request():
    cache = manager(capacity=400, step=8)
    window_group = cache.paged[cache.locate(4)[1]]
    full_group = cache.paged[cache.locate(1)[1]]
    assert cache.pages_for(full_group, 400) == 100
    assert cache.pages_for(window_group, 400) == 6            # ceil((9 + 8) / 4) + 1
    cache.open("a", reserve_tokens=400)
    length = 0
    while length < 400:
        step = min(8, 400 - length)
        cache.grow("a", step)
        cache.advance("a", step)
        length += step
        assert cache.get("a").live[cache.locate(4)[1]] <= 6
        cache.check()
    cache.close("a")
    cache.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    """Requests open, grow by random portions, advance, sometimes fail for lack of pages, and
    close in random order; after every operation every page and slot is either free or held
    by exactly one request."""
    rng = random.Random(seed)
    cache = manager(capacity=96, page=4, requests=5, step=16)
    live, next_id = {}, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.2 and len(live) < 5:
            reserve = rng.choice([None, None, rng.randint(1, 60)])
            try:
                cache.open(next_id, reserve_tokens=reserve)
                live[next_id] = reserve
            except CacheCapacityError:
                assert next_id not in cache
            next_id += 1
        elif action < 0.85 and live:
            request = rng.choice(list(live))
            portion = rng.randint(1, 16)
            try:
                cache.grow(request, portion)
                cache.advance(request, portion)
            except CacheCapacityError:
                pass
        elif live:
            request = rng.choice(list(live))
            cache.close(request)
            del live[request]
        cache.check()
        for request, reserve in live.items():
            if reserve is not None:
                assert cache.get(request).length <= reserve
    cache.close_all()
    cache.check()
    stats = cache.stats()
    assert stats.pages_free == stats.pages_total and stats.slots_free == stats.slots_total
    assert all(p == 0 for p in stats.pages_promised)


def test_slots_are_zeroed_when_handed_out():
    cache = manager(allocate=True)
    first = cache.open("a")
    slot = first.slots[0]
    cache.states[0].storage[:, slot] = 7.0
    cache.close("a")
    again = cache.open("b")
    assert again.slots[0] == slot
    assert float(cache.states[0].storage[:, slot].abs().sum()) == 0.0
    for _ in range(3):
        cache.open(object())
    with pytest.raises(CacheCapacityError):
        cache.open("one too many")
