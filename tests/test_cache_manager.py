"""Cache manager bookkeeping: no page lost, held twice or freed twice (no GPU)."""
import random

import pytest

from infero_b200.cache import CacheManager, GroupSpec, OutOfPages, OutOfSlots


def test_allocator_is_all_or_nothing_and_never_frees_twice():
    """The allocator generation uses (csrc/host_cache.cpp) through the manager: lowest pages first, a
    request that does not fit takes nothing, a page that came back is handed out again, and closing
    a request twice gives nothing back twice."""
    m = CacheManager([GroupSpec(None)], num_pages=4, page_size=16, max_requests=3)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 48)
    m.commit(a, 48)
    assert a.tables == [[0, 1, 2]] and m.free_pages(0) == 1
    with pytest.raises(OutOfPages) as e:
        m.reserve(b, 17)
    assert (e.value.group, e.value.wanted, e.value.free) == (0, 2, 1)
    assert m.free_pages(0) == 1 and b.tables == [[]]
    m.reserve(b, 16)
    m.commit(b, 16)
    assert b.tables == [[3]] and m.allocators[0].held_pages() == [0, 1, 2, 3]
    m.close("a")
    assert m.free_pages(0) == 3 and m.allocators[0].held_pages() == [3]
    with pytest.raises(KeyError):
        m.close("a")
    assert m._L.infero_cache_close(m._h, a.slot) != 0        # the native side refuses a slot that is not open
    assert m.free_pages(0) == 3
    m.check()
    c = m.open("c")
    m.reserve(c, 33)
    assert sorted(c.tables[0]) == [0, 1, 2] and m.pages_reused == 3
    m.check()


def test_every_group_has_a_pool_of_its_own_size():
    """A window group with far fewer pages than the all-keys group: long requests run in portions, the
    window pages come back as the window passes, and only the group that is short refuses."""
    W, P = 32, 16
    m = CacheManager([GroupSpec(None), GroupSpec(W)], num_pages=[40, 6], page_size=P, max_requests=2)
    assert [a.num_pages for a in m.allocators] == [40, 6] and m.num_pages == 40
    a = m.open("a")
    for n in [40, 40, 40, 40, 1, 1, 30, 64]:
        m.reserve(a, n)
        m.commit(a, n)
        m.check()
        assert m.allocators[1].num_pages - m.free_pages(1) <= -(-W // P) + 1
    assert a.length == 256 and m.free_pages(0) == 40 - 16 and m.pages_reclaimed >= 13
    with pytest.raises(OutOfPages) as e:
        m.reserve(a, 97)                      # the window group cannot hold a portion that long
    assert e.value.group == 1 and m.free_pages(0) == 24
    b = m.open("b")
    with pytest.raises(OutOfPages) as e:
        m.reserve(b, 25 * P)                  # and here the all-keys group is the one that is short
    assert e.value.group == 0
    m.close("a")
    m.close("b")
    assert [m.free_pages(g) for g in (0, 1)] == [40, 6]
    m.check()


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


def test_the_table_copy_for_the_device_marks_released_pages():
    m = CacheManager([GroupSpec(16)], num_pages=8, page_size=16, max_requests=2, max_blocks=6)
    a = m.open("a")
    m.reserve(a, 40)
    m.commit(a, 40)
    t = m._mirror(0)[a.slot]
    # the next query, at position 40, sees keys 25 .. 40: page 0 (keys 0 .. 15) went back
    assert t.shape == (6,) and t[0] == -1 and t[1] >= 0 and t[2] >= 0 and t[3] == -1
    assert a.tables == [[-1, int(t[1]), int(t[2])]] and a.first_live == [1]


@pytest.mark.parametrize("seed", range(12))
def test_random_orders_of_requests_keep_every_invariant(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(None), GroupSpec(rng.choice([16, 24, 48, 100]))]
    P = rng.choice([16, 32, 64])
    pools = [rng.randint(6, 24), rng.randint(6, 24)] if seed % 2 else rng.randint(6, 24)
    m = CacheManager(groups, num_pages=pools, page_size=P, max_requests=4)
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
        elif op < 0.92 and live:
            rc = live[rng.choice(list(live))]
            before = (rc.length, [a.num_free for a in m.allocators])
            try:
                m.truncate(rc, max(0, rc.length - rng.choice([0, 1, 5, 40])))
            except ValueError:
                assert (rc.length, [a.num_free for a in m.allocators]) == before
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


def test_storage_keeps_keys_and_values_at_their_own_widths_and_pools():
    """Keys and values are two arrays per group (a mixer may cache values wider or narrower than its
    keys), and every group's arrays have its own number of pages."""
    import torch
    from infero_b200.cache import CacheStorage, plan_group_pages
    from infero_b200.cache.storage import group_cache_slots, window_pool_pages
    from infero_b200.parts.base import KvCacheSpec
    specs = {0: KvCacheSpec(2, 16, None), 1: KvCacheSpec(2, 16, 32), 2: KvCacheSpec(2, 16, 32),
             3: KvCacheSpec(3, 8, None, v_head_dim=24)}
    groups, where = group_cache_slots(specs)
    assert len(groups) == 3 and where[2] == (1, 1)
    pages = plan_group_pages(groups, 500, 16, max_requests=4, max_batch_tokens=64)
    assert pages == [500, window_pool_pages(32, 16, 4, 64), 500] and pages[1] == 4 * 5 + 4
    st = CacheStorage(specs, {}, [n + 1 for n in pages], 16, 5, torch.float32, "cpu")
    assert st.layer_kv(0).k.shape == (501, 2, 16, 16) and st.layer_kv(2).v.shape == (25, 2, 16, 16)
    assert st.layer_kv(3).k.shape == (501, 3, 16, 8) and st.layer_kv(3).v.shape == (501, 3, 16, 24)
    assert st.bytes_per_token() == 4 * (2 * 2 * 16 * 3 + 3 * (8 + 24))
    assert st.bytes() == 4 * 16 * (501 * 64 + 2 * 25 * 64 + 501 * 96)


def test_truncate_gives_back_the_tail_and_refuses_what_a_window_lost():
    m = CacheManager([GroupSpec(None), GroupSpec(32)], num_pages=[16, 8], page_size=16, max_requests=2)
    a = m.open("a")
    m.reserve(a, 70)
    m.commit(a, 70)                                   # window pages 0 and 1 (keys 0 .. 31) went back
    assert a.tables[1][:2] == [-1, -1] and m.free_pages(0) == 11
    m.truncate(a, 65)                                 # a query at 65 sees keys 34 .. 65: still all held
    assert a.length == 65 and len(a.tables[0]) == 5 and m.free_pages(0) == 11
    m.truncate(a, 64)                                 # the fifth page is behind the end now
    assert len(a.tables[0]) == 4 and len(a.tables[1]) == 4 and m.free_pages(0) == 12
    m.check()
    with pytest.raises(ValueError, match="window"):
        m.truncate(a, 50)                             # would see keys 19 .. 50, and page 1 is gone
    with pytest.raises(ValueError):
        m.truncate(a, 65)                             # nothing to cut
    assert a.length == 64
    m.reserve(a, 3)
    with pytest.raises(ValueError):
        m.truncate(a, 60)                             # a step is in flight
    m.commit(a, 3)
    b = m.open("b")
    m.reserve(b, 40)
    m.commit(b, 40)
    m.truncate(b, 0)
    assert b.length == 0 and b.fresh and b.tables == [[], []]
    m.check()
    m.close("a"); m.close("b")
    assert [m.free_pages(g) for g in (0, 1)] == [16, 8]
