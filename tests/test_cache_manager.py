"""Cache manager bookkeeping: no page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from infero_b200.cache import CacheManager, GroupSpec, OutOfPages, OutOfSlots, PageAllocator


def test_allocator_is_all_or_nothing_and_refuses_double_free():
    a = PageAllocator(4)
    got = a.alloc(3)
    assert got == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.alloc(2)
    assert a.num_free == 1
    a.free([1])
    with pytest.raises(AssertionError):
        a.free([1])
    with pytest.raises(AssertionError):
        a.free([3])
    assert a.alloc(2) == [1, 3]


def test_pages_follow_the_length_and_come_back_on_close():
    m = CacheManager([GroupSpec(None)], num_pages=8, page_size=16, max_requests=2)
    rc = m.open("a")
    m.reserve(rc, 17)
    assert len(rc.tables[0]) == 2
    m.commit(rc, 17)
    m.reserve(rc, 15)
    assert len(rc.tables[0]) == 2          # 32 tokens still fit two pages
    m.commit(rc, 15)
    m.reserve(rc, 1)
    assert len(rc.tables[0]) == 3
    m.commit(rc, 1)
    m.check()
    m.close("a")
    assert m.free_pages(0) == 8
    m.check()


def test_reserve_takes_nothing_when_one_group_is_short():
    m = CacheManager([GroupSpec(None), GroupSpec(32)], num_pages=4, page_size=16, max_requests=2)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 48)
    m.commit(a, 48)
    with pytest.raises(OutOfPages):
        m.reserve(b, 40)
    assert b.tables == [[], []] and b.reserved == 0
    m.check()


def test_window_group_gives_pages_back_as_the_window_passes():
    W, P = 48, 16
    m = CacheManager([GroupSpec(None), GroupSpec(W)], num_pages=32, page_size=P, max_requests=1)
    rc = m.open("a")
    length = 0
    for n in [5, 30, 1, 1, 64, 2, 100, 1]:
        m.reserve(rc, n)
        m.commit(rc, n)
        length += n
        m.check()
        full, win = rc.tables
        assert all(p >= 0 for p in full) and len(full) == -(-length // P)
        for k, p in enumerate(win):
            last_pos = k * P + P - 1
            dead = last_pos <= length - W          # the next query is at `length`; it sees j > length - W
            assert (p < 0) == dead, (length, k, p)
    assert m.pages_reclaimed > 0
    m.close("a")
    assert m.free_pages(0) == 32 and m.free_pages(1) == 32


def test_state_slots_are_unique_and_bounded():
    m = CacheManager([GroupSpec(None)], num_pages=4, page_size=16, max_requests=3)
    slots = {m.open(i).slot for i in range(3)}
    assert slots == {0, 1, 2}
    with pytest.raises(OutOfSlots):
        m.open("x")
    m.close(1)
    assert m.open("y").slot == 1 and m.get("y").fresh
    with pytest.raises(KeyError):
        m.open("y")


def test_abort_returns_reserved_pages_only():
    m = CacheManager([GroupSpec(None)], num_pages=8, page_size=16, max_requests=1)
    rc = m.open("a")
    m.reserve(rc, 20)
    m.commit(rc, 20)
    m.reserve(rc, 40)
    assert m.free_pages(0) == 4
    m.abort_reservation(rc)
    assert m.free_pages(0) == 6 and rc.length == 20 and len(rc.tables[0]) == 2
    m.check()


def test_block_table_array_marks_released_pages():
    m = CacheManager([GroupSpec(16)], num_pages=8, page_size=16, max_requests=2)
    a = m.open("a")
    m.reserve(a, 40)
    m.commit(a, 40)
    t = m.block_table_array(0, [a], 6)
    assert t.shape == (1, 6) and t[0, 0] == -1 and t[0, 2] >= 0 and t[0, 3] == -1


@pytest.mark.parametrize("seed", range(12))
def test_random_orders_of_requests_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(None), GroupSpec(rng.choice([16, 24, 48, 100]))]
    P = rng.choice([16, 32, 64])
    m = CacheManager(groups, num_pages=rng.randint(6, 24), page_size=P, max_requests=4)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            live[next_id] = m.open(next_id)
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            n = rng.choice([1, 1, 1, 2, 7, 16, 33, 70])
            before = [a.num_free for a in m.allocators]
            try:
                m.reserve(rc, n)
            except OutOfPages:
                assert [a.num_free for a in m.allocators] == before
                if rng.random() < 0.5:
                    m.close(rid)
                    del live[rid]
                m.check()
                continue
            if rng.random() < 0.1:
                m.abort_reservation(rc)
            else:
                m.commit(rc, n)
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check()
    for rid in list(live):
        m.close(rid)
    m.check()
    assert all(a.num_free == a.num_pages for a in m.allocators)
    assert m.pages_reused > 0
