"""The cache's bookkeeping on the host: slots and pages are never lost, held twice or freed
twice; groups with a window give pages back; everything is reusable after a batch ends."""

import random

import pytest

from thing_htn_2026_b200.cache import CacheBook, CacheFull, CacheStateError, GroupBook, IdAllocator


def test_allocator_hands_out_each_id_once():
    a = IdAllocator(5, "slot")
    got = a.take(3)
    assert got == [0, 1, 2] and a.n_free == 2 and a.n_held == 3
    with pytest.raises(CacheFull):
        a.take(3)
    assert a.n_free == 2                     # a refused request takes nothing
    a.give_back([1])
    assert a.take(1) == [1]                  # lowest free id first: reuse
    a.check()


def test_allocator_refuses_double_free():
    a = IdAllocator(4, "page")
    ids = a.take(2)
    a.give_back(ids)
    with pytest.raises(CacheStateError, match="not held"):
        a.give_back([ids[0]])
    with pytest.raises(CacheStateError, match="not held"):
        a.give_back([3])                     # never taken
    b = a.take(2)
    with pytest.raises(CacheStateError, match="freed twice"):
        a.give_back([b[0], b[0]])
    a.check()


def book(n_pages=8, window=None, max_slots=4, max_pages_per_seq=8):
    return CacheBook([GroupBook(window, n_pages)], 64, max_slots, max_pages_per_seq)


def test_pages_follow_lengths():
    b = book()
    s0, s1 = b.open(), b.open()
    updates = b.prepare([s0, s1], [65, 1])
    assert sorted((slot, logical) for _, slot, logical, _ in updates) == [(s0, 0), (s0, 1), (s1, 0)]
    assert len({physical for *_, physical in updates}) == 3
    b.commit([s0, s1], [65, 1])
    assert (b.length(s0), b.length(s1)) == (65, 1) and b.tokens_held() == 128 + 64
    assert b.prepare([s0, s1], [63, 63]) == []               # room left in the mapped pages
    b.commit([s0, s1], [63, 63])
    assert [u[1:3] for u in b.prepare([s0, s1], [1, 1])] == [(s0, 2), (s1, 1)]
    b.check()


def test_prepare_is_all_or_nothing():
    b = book(n_pages=3)
    s0, s1 = b.open(), b.open()
    with pytest.raises(CacheFull, match="needs 4 more pages"):
        b.prepare([s0, s1], [128, 100])
    assert b.pages[0].n_free == 3 and b.pages_of(0, s0) == {}
    with pytest.raises(CacheStateError, match="twice in one step"):
        b.prepare([s0, s0], [1, 1])
    with pytest.raises(CacheFull, match="longest sequence"):
        book(n_pages=100, max_pages_per_seq=2).prepare([0], [129]) if False else _too_long()
    b.check()


def _too_long():
    b = book(n_pages=100, max_pages_per_seq=2)
    s = b.open()
    b.prepare([s], [129])


def test_close_gives_everything_back_and_refuses_twice():
    b = book()
    s = b.open()
    b.prepare([s], [200])
    b.commit([s], [200])
    updates = b.close(s)
    assert sorted(u[2] for u in updates) == [0, 1, 2, 3] and all(u[3] == -1 for u in updates)
    assert b.pages[0].n_free == 8 and b.slots.n_free == 4 and b.tokens_held() == 0
    with pytest.raises(CacheStateError, match="not open"):
        b.close(s)
    with pytest.raises(CacheStateError, match="not open"):
        b.length(s)
    assert b.open() == s                       # the slot is used again
    b.check()


def test_windowed_group_keeps_only_what_can_be_read():
    b = CacheBook([GroupBook(None, 16), GroupBook(70, 16)], 64, 2, 16)
    s = b.open()
    b.prepare([s], [300])                      # a long prompt holds all its pages during the step
    assert len(b.pages_of(1, s)) == 5
    dropped = b.commit([s], [300])
    # next query is at 300 and reads keys > 230: pages 0..2 (positions < 192) are gone
    assert sorted(u[2] for u in dropped if u[0] == 1) == [0, 1, 2] and all(u[3] == -1 for u in dropped)
    assert sorted(b.pages_of(1, s)) == [3, 4] and len(b.pages_of(0, s)) == 5
    for _ in range(200):                       # single-token steps: never more than 3 pages
        b.prepare([s], [1])
        b.commit([s], [1])
        assert len(b.pages_of(1, s)) <= 3
    assert len(b.pages_of(0, s)) == 8
    b.check()
    b.close(s)
    assert b.pages[0].n_free == 16 and b.pages[1].n_free == 16


def test_random_batches_never_lose_a_page():
    rng = random.Random(0)
    b = CacheBook([GroupBook(None, 40), GroupBook(100, 40)], 64, 6, 12)
    live = {}
    for _ in range(400):
        action = rng.random()
        if action < 0.3 and b.slots.n_free:
            live[b.open()] = True
        elif action < 0.45 and live:
            slot = rng.choice(list(live))
            b.close(slot)
            del live[slot]
        elif live:
            slots = rng.sample(list(live), rng.randint(1, len(live)))
            counts = [rng.choice([1, 1, 1, 17, 64, 90]) for _ in slots]
            try:
                b.prepare(slots, counts)
            except CacheFull:
                continue
            b.commit(slots, counts)
        b.check()
    for slot in list(live):
        b.close(slot)
    b.check()
    assert b.tokens_held() == 0 and all(p.n_free == 40 for p in b.pages) and b.slots.n_free == 6
