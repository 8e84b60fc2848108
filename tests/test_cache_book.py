"""Slots and pages on the host: nothing lost, held twice or freed twice (no GPU)."""
import random

import pytest

from agave_b200.cache.book import (PAGE, CacheBook, CacheError, CacheFull, PagePool,
                                   SlotAllocator, plan_groups, round_up)
from agave_b200.parts.base import KVRequest, StateRequest


def test_slots_are_unique_and_reused():
    a = SlotAllocator(4)
    got = [a.acquire() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheFull):
        a.acquire()
    a.release(2)
    with pytest.raises(CacheError):
        a.release(2)                       # freed twice
    with pytest.raises(CacheError):
        a.release(7)                       # never acquired
    assert a.acquire() == 2 and a.n_free == 0


def test_pages_all_or_nothing():
    p = PagePool(5)
    x = p.alloc(3)
    with pytest.raises(CacheFull):
        p.alloc(3)
    assert p.n_free == 2                   # the failed request took nothing
    p.free(x)
    with pytest.raises(CacheError):
        p.free(x[:1])
    assert p.n_free == 5


def _book(max_tokens=1024, max_seq_len=512, n_slots=8, window=100):
    reqs = [KVRequest(2, 32, window), KVRequest(2, 32, None), KVRequest(2, 32, window),
            StateRequest(8), None]
    groups, where = plan_groups(reqs, max_tokens, max_seq_len, n_slots)
    return CacheBook(groups, n_slots, max_seq_len), groups, where


def test_groups_by_need():
    book, groups, where = _book()
    assert len(groups) == 2
    win = groups[where[0][0]]
    full = groups[where[1][0]]
    assert win.window == 100 and win.cap == 128 and win.entries == [0, 2]
    assert full.window is None and full.cap == 512 and full.entries == [1]
    assert where[2] == (where[0][0], 1) and 3 not in where and 4 not in where
    assert full.n_pages == 1024 // PAGE


def test_window_bigger_than_the_cache_is_a_full_group():
    groups, where = plan_groups([KVRequest(1, 16, 4096), KVRequest(1, 16, None)], 1024, 512, 4)
    assert len(groups) == 1 and groups[0].window is None


def test_ring_stops_growing_and_full_group_grows():
    book, groups, where = _book()
    s = book.acquire()
    gi_win, gi_full = where[0][0], where[1][0]
    for n in (1, 64, 65, 128, 129, 400):
        book.reserve(s, n)
        book.set_length(s, n)
        assert len(book.pages[s][gi_full]) == round_up(n, PAGE) // PAGE
        assert len(book.pages[s][gi_win]) == min(round_up(n, PAGE), 128) // PAGE
    with pytest.raises(CacheFull):
        book.reserve(s, 513)
    book.release(s)
    assert all(p.n_free == p.n_pages for p in book.pools)


def test_random_lifecycles_conserve_slots_and_pages():
    rng = random.Random(0)
    book, groups, where = _book(max_tokens=2048, max_seq_len=512, n_slots=6)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and book.slots.n_free:
            s = book.acquire()
            assert s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 1, 70])
            try:
                book.reserve(s, n)
                book.set_length(s, n)
                live[s] = n
            except CacheFull:
                pass
        elif live:
            s = rng.choice(list(live))
            book.release(s)
            del live[s]
        # invariants: every page held exactly once, by a live slot
        for gi, pool in enumerate(book.pools):
            held = [p for s in live for p in book.pages[s][gi]]
            assert len(held) == len(set(held)) == pool.n_pages - pool.n_free
        assert book.slots.held == frozenset(live)
        assert book.live_tokens() == sum(round_up(n, PAGE) for n in live.values())
    for s in list(live):
        book.release(s)
    assert book.slots.n_free == 6 and all(p.n_free == p.n_pages for p in book.pools)
    with pytest.raises(CacheError):
        book.release(0)


def test_trim_gives_back_what_a_step_that_did_not_run_reserved():
    book, groups, where = _book()
    s = book.acquire()
    book.reserve(s, 70)
    book.set_length(s, 70)
    held = [len(p) for p in book.pages[s]]
    free = [p.n_free for p in book.pools]
    book.reserve(s, 400)                       # a step that is then refused
    assert [p.n_free for p in book.pools] != free
    book.dirty.clear()
    book.trim(s)
    assert [len(p) for p in book.pages[s]] == held and [p.n_free for p in book.pools] == free
    assert s in book.dirty                     # the table row changed again
    book.trim(s)                               # nothing more to give back
    assert [p.n_free for p in book.pools] == free
    book.release(s)
    assert all(p.n_free == p.n_pages for p in book.pools)
    with pytest.raises(CacheError):
        book.trim(s)
