"""The cache's host bookkeeping: no slot or page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from rust_inference_b200.cache.pager import CacheError, CacheFull, SlotPager


def test_slots_are_handed_out_once_and_reused():
    p = SlotPager(n_slots=3, n_pages=8, page_size=64, max_seq_len=512)
    a, b, c = p.alloc_slot(), p.alloc_slot(), p.alloc_slot()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheFull):
        p.alloc_slot()
    p.free_slot(b)
    assert p.alloc_slot() == b                       # a freed slot is used again
    p.audit()


def test_free_twice_and_unknown_slots_are_errors():
    p = SlotPager(2, 4, 64, 256)
    s = p.alloc_slot()
    p.free_slot(s)
    with pytest.raises(CacheError, match="not in use"):
        p.free_slot(s)
    with pytest.raises(CacheError, match="not in use"):
        p.length(1)
    with pytest.raises(CacheError, match="does not exist"):
        p.reserve(7, 10)
    p.audit()


def test_pages_follow_lengths_and_return_on_free():
    p = SlotPager(4, 6, 64, 1024)
    s, t = p.alloc_slot(), p.alloc_slot()
    assert p.reserve(s, 1) != [] and len(p.pages(s)) == 1
    assert p.reserve(s, 64) == []                    # still the first page
    assert len(p.reserve(s, 65)) == 1                # the 65th position opens a second page
    p.set_length(s, 65)
    p.reserve(t, 200)
    assert len(p.pages(t)) == 4 and p.free_page_count() == 0
    assert set(p.pages(s)).isdisjoint(p.pages(t))    # no page held twice
    with pytest.raises(CacheFull, match="cache is full"):
        p.reserve(s, 129)
    p.free_slot(t)
    assert p.free_page_count() == 4
    assert len(p.reserve(s, 129)) == 1
    p.audit()
    with pytest.raises(CacheError, match="exceeds its reserved pages"):
        p.set_length(s, 500)


def test_a_fresh_slot_starts_empty():
    p = SlotPager(1, 4, 64, 256)
    s = p.alloc_slot()
    p.reserve(s, 100)
    p.set_length(s, 100)
    p.free_slot(s)
    s2 = p.alloc_slot()
    assert s2 == s and p.length(s2) == 0 and p.pages(s2) == []


def test_max_seq_len_is_a_finish_not_a_fault():
    p = SlotPager(1, 100, 64, 130)
    s = p.alloc_slot()
    p.reserve(s, 130)
    with pytest.raises(CacheFull, match="max_seq_len"):
        p.reserve(s, 131)
    p.audit()


def test_reserve_many_is_all_or_nothing():
    p = SlotPager(3, 4, 64, 1024)
    a, b = p.alloc_slot(), p.alloc_slot()
    with pytest.raises(CacheFull):
        p.reserve_many([(a, 128), (b, 192)])         # 2 + 3 pages > 4
    assert p.free_page_count() == 4 and p.pages(a) == [] and p.pages(b) == []
    p.reserve_many([(a, 128), (b, 128)])
    assert p.free_page_count() == 0
    p.audit()


def test_a_step_moves_all_its_slots_or_none():
    p = SlotPager(3, 8, 64, 512)
    a, b = p.alloc_slot(), p.alloc_slot()
    p.reserve_many([(a, 100), (b, 10)])
    p.advance([a, b], [100, 10])
    assert p.lengths([b, a]) == [10, 100]
    with pytest.raises(CacheError, match="exceeds its reserved pages"):
        p.advance([a, b], [1, 60])                   # b has one page: 70 positions do not fit
    assert p.lengths([a, b]) == [100, 10]            # a did not move either
    with pytest.raises(CacheError, match="not in use"):
        p.lengths([a, 2])
    p.audit()


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    p = SlotPager(n_slots=5, n_pages=40, page_size=64, max_seq_len=1000)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            s = p.alloc_slot()
            assert s not in live
            live[s] = 0
        elif op < 0.45 and live:
            s = rng.choice(list(live))
            p.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 150)
            try:
                p.reserve(s, new)
                p.set_length(s, new)
                live[s] = new
            except CacheFull:
                pass
        p.audit()
        assert sorted(live) == p.live_slots()
        for s, n in live.items():
            assert p.length(s) == n and len(p.pages(s)) >= -(-n // 64)
    for s in list(live):
        p.free_slot(s)
    p.audit()
    assert p.free_slot_count() == 5 and p.free_page_count() == 40
