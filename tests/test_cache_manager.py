"""The host cache manager: page pools, groups with a window, promises, state slots.

Fixed vectors follow the reference's own pool tests (src/engine/kvcache/pool.rs:487-548,
src/scheduler/prefill.rs:612-624); the random runs check that no page is ever lost, held
twice or freed twice.
"""
import random

import pytest

from llm_infer_rust_b200.cache.paged import cache_budget_bytes
from llm_infer_rust_b200.kernels.build import load_host_runtime

rt = load_host_runtime()


def manager(pages, page_size=4, window=0, slots=8):
    if isinstance(pages, int):
        pages, window = [pages], [window]
    return rt.CacheManager([rt.GroupSpec(page_size, n, w) for n, w in zip(pages, window)], slots)


def test_pool_hands_out_from_the_top_and_refuses_a_second_free():
    pool = rt.PagePool(10)
    assert [pool.alloc() for _ in range(3)] == [10, 9, 8]
    assert [pool.alloc() for _ in range(2)] == [7, 6]
    assert pool.free_count() == 5
    assert pool.release(9) and not pool.release(9)          # freeing twice is refused
    assert not pool.release(0) and not pool.release(11) and not pool.release(3)   # sink, foreign, not held
    assert pool.alloc() == 9                                # the page just freed is used again first
    small = rt.PagePool(3)
    assert [small.alloc() for _ in range(4)] == [3, 2, 1, -1]
    assert 0 not in small.free_list()


def test_budget_formula():
    assert cache_budget_bytes(600, 1000, 0.9) == 500
    assert cache_budget_bytes(100, 1000, 0.9) == 0


def test_grow_advance_release_and_slots():
    m = manager(6, page_size=4)
    assert m.open(1) == rt.Acquire.Ready and m.state_slot(1) == 1
    assert m.grow(1, 5) and m.block_table(1, 0) == [6, 5] and m.length(1) == 0
    m.advance(1, 5)
    assert m.length(1) == 5 and m.slot_of(1, 0, 0) == 24 and m.slot_of(1, 0, 4) == 20 and m.slot_of(1, 0, 8) == -1
    assert m.open(2) == rt.Acquire.Ready and m.state_slot(2) == 2
    assert m.grow(2, 16) and m.free_pages(0) == 0
    assert not m.grow(1, 9)                                  # nothing left, and nothing changed
    assert m.block_table(1, 0) == [6, 5] and m.check() == ""
    assert m.release(2) and not m.release(2)                 # a second release is a no-op
    assert m.grow(1, 9) and m.block_table(1, 0) == [6, 5, 1]   # pages come back in LIFO order
    assert m.open(3) == rt.Acquire.Ready and m.state_slot(3) == 2    # the slot too
    assert m.check() == ""
    with pytest.raises(Exception):
        m.open(3)


def test_promise_at_admission_keeps_pages_for_a_running_request():
    m = manager(4, page_size=2)
    # capacity excludes the last sampled token: prompt 2, one new token, max_seq 3 -> 1 page
    assert m.pages_needed(0, min(2 + 1 - 1, 3), 8) == 1
    assert m.acquire(1, 6, 8) == rt.Acquire.Ready            # 3 pages promised
    assert m.unpromised_pages(0) == 1 and m.free_pages(0) == 4
    assert m.acquire(2, 4, 8) == rt.Acquire.DeferredMemory   # would need 2
    assert m.acquire(2, 10, 8) == rt.Acquire.Impossible      # more than the pool has
    assert m.acquire(2, 2, 8) == rt.Acquire.Ready
    assert m.grow(2, 2) and not m.grow(2, 3)                 # beyond its promise and nothing is unpromised
    assert m.grow(1, 6) and m.free_pages(0) == 0 and m.check() == ""
    m.release(1)
    assert m.free_pages(0) == 3 and m.unpromised_pages(0) == 3
    m.release(2)
    assert m.free_pages(0) == 4 and m.check() == ""


def test_state_slots_run_out_before_pages():
    m = manager(50, slots=2)
    assert m.open(1) == rt.Acquire.Ready and m.open(2) == rt.Acquire.Ready
    assert m.open(3) == rt.Acquire.DeferredSlots
    m.release(1)
    assert m.open(3) == rt.Acquire.Ready and m.state_slot(3) == 1


def test_a_window_gives_pages_back_while_the_request_runs():
    m = manager([8, 8], page_size=4, window=[0, 6])
    m.open(1)
    assert m.grow(1, 10)
    m.advance(1, 10)
    # next query at position >= 10 reads keys > 10 - 6 = 4: page 0 (positions 0..3) is passed
    assert m.pages_held(1, 0) == 3 and m.pages_held(1, 1) == 2 and m.first_live_page(1, 1) == 1
    assert m.block_table(1, 1)[0] == 0 and m.slot_of(1, 1, 3) == -1 and m.slot_of(1, 1, 4) > 0
    for length in range(11, 33):
        assert m.grow(1, length)
        m.advance(1, length)
        assert m.pages_held(1, 1) <= 3 and m.check() == ""
    assert m.pages_held(1, 0) == 8
    assert not m.grow(1, 33)                                 # the full group is exhausted
    m.release(1)
    assert m.free_pages(0) == 8 and m.free_pages(1) == 8 and m.check() == ""


def test_pages_needed_with_a_window():
    m = manager([100, 100], page_size=4, window=[0, 6])
    assert m.pages_needed(0, 40, 1) == 10
    assert m.pages_needed(1, 40, 1) == 3                     # ceil((6 + 1 - 1) / 4) + 1
    assert m.pages_needed(1, 40, 16) == 7                    # ceil((6 + 16 - 1) / 4) + 1
    assert m.pages_needed(1, 5, 16) == 2                     # never more than all its tokens


def test_a_windowed_promise_is_enough_for_any_cutting():
    """A request admitted with a promise for (capacity, step bound) never fails to grow."""
    rng = random.Random(7)
    for trial in range(60):
        P, W, step = rng.choice([2, 4, 8]), rng.randint(1, 20), rng.randint(1, 12)
        cap = rng.randint(1, 90)
        m = manager([64, 64], page_size=P, window=[0, W])
        assert m.acquire(1, cap, step) == rt.Acquire.Ready
        # a greedy competitor takes everything that is not promised
        m.open(2)
        n = 0
        while m.grow(2, n + 1):
            n += 1
        length = 0
        while length < cap:
            take = min(rng.randint(1, step), cap - length)
            assert m.grow(1, length + take), (trial, P, W, step, cap, length, take)
            length += take
            m.advance(1, length)
            assert m.check() == ""
        m.release(1)
        m.release(2)
        assert m.free_pages(0) == 64 and m.free_pages(1) == 64 and m.check() == ""


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    P = rng.choice([1, 4, 16])
    windows = [0, rng.randint(1, 40)] if seed % 2 else [0]
    pages = [rng.randint(8, 40) for _ in windows]
    m = manager(pages, page_size=P, window=windows, slots=5)
    live = {}
    next_id = 1
    for _ in range(1500):
        op = rng.random()
        if op < 0.25 and len(live) < 6:
            how = rng.random()
            if how < 0.5:
                got = m.open(next_id)
            else:
                got = m.acquire(next_id, rng.randint(1, 120), rng.randint(1, 30))
            if got == rt.Acquire.Ready:
                live[next_id] = 0
            else:
                assert not m.has(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            new_len = live[rid] + rng.randint(1, 30)
            before = [m.free_pages(g) for g in range(len(pages))]
            if m.grow(rid, new_len):
                m.advance(rid, new_len)
                live[rid] = new_len
                for g, w in enumerate(windows):              # every readable position has a page
                    lo = 0 if w == 0 else max(0, new_len - w + 1)
                    assert all(m.slot_of(rid, g, p) >= P for p in range(lo, new_len))
            else:
                assert before == [m.free_pages(g) for g in range(len(pages))]
        elif live:
            rid = rng.choice(list(live))
            assert m.release(rid) and not m.release(rid)
            del live[rid]
        assert m.check() == "", m.check()
        assert m.live_requests() == len(live)
    for rid in list(live):
        m.release(rid)
    assert [m.free_pages(g) for g in range(len(pages))] == pages and m.free_state_slots() == 5
    assert m.check() == ""


def test_growth_of_a_whole_step_is_all_or_nothing():
    """A step's entries get their pages together or not at all: an entry that does not fit leaves the ones
    before it as they were (pages that only a promise covers count for the request that holds the promise)."""
    m = manager(6, page_size=4)
    for rid in (1, 2, 3):
        assert m.open(rid) == rt.Acquire.Ready
    assert m.grow_all([1, 2], [8, 8]) == -1 and m.free_pages(0) == 2
    before = [list(m.block_table(r, 0)) for r in (1, 2, 3)]
    assert m.grow_all([1, 3, 2], [12, 5, 9]) == 1            # 1 + 2 + 1 pages wanted, two are free: request 3 is short
    assert [list(m.block_table(r, 0)) for r in (1, 2, 3)] == before and m.free_pages(0) == 2 and m.check() == ""
    assert m.grow_all([1, 3], [12, 3]) == -1 and m.free_pages(0) == 0 and m.check() == ""
    with pytest.raises(Exception):
        m.grow_all([1, 1], [13, 14])                         # a request twice in one step
    with pytest.raises(Exception):
        m.grow_all([1], [13, 14])
    # with a promise: request 5's promised pages are its own, request 4 cannot take them
    p = manager(4, page_size=2)
    assert p.acquire(5, 6, 6) == rt.Acquire.Ready and p.open(4) == rt.Acquire.Ready
    assert p.grow_all([4, 5], [4, 6]) == 0 and p.free_pages(0) == 4          # 4 wants two pages, one is unpromised
    assert p.grow_all([4, 5], [2, 6]) == -1 and p.free_pages(0) == 0 and p.check() == ""
