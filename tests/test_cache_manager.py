"""The cache manager on the host: no page lost, held twice or freed twice, under random
orders of requests; groups with a window give pages back; slots are zeroed and reused."""

import random

import pytest
import torch

from acorninfer_b200.cache.manager import CacheManager
from acorninfer_b200.cache.pools import IdPool, PoolExhausted
from acorninfer_b200.parts.base import KVNeeds, StateNeeds


def manager(num_pages=16, page_size=4, window=None, slots=4, allocate=False, two_groups=False):
    needs = {0: KVNeeds(2, 8, None), 1: KVNeeds(2, 8, None)}
    if two_groups or window:
        needs[2] = KVNeeds(2, 8, window or 6)
    return CacheManager(needs, {}, num_pages, page_size, slots, dtype=torch.float32, device="cpu", allocate=allocate)


def test_pool_is_lifo_and_refuses_double_free():
    p = IdPool(4)
    a = p.allocate(2)
    assert a == [0, 1] and p.num_free == 2
    p.free([1])
    assert p.allocate(1) == [1]                       # the page just given back is used again first
    with pytest.raises(ValueError):
        p.free([3])                                   # never allocated
    p.free([0])
    with pytest.raises(ValueError):
        p.free([0])                                   # freed twice
    with pytest.raises(PoolExhausted):
        p.allocate(4)
    assert p.num_free == 3                            # all or nothing: nothing was taken
    p.free([1])
    p.assert_balanced()


def test_layers_with_equal_needs_share_a_group_and_a_page_id():
    m = manager(two_groups=True)
    assert len(m.groups) == 2
    assert m.entry_group[0] == (0, 0) and m.entry_group[1] == (0, 1) and m.entry_group[2] == (1, 0)


def test_extend_commit_close():
    m = manager(num_pages=8, page_size=4)
    rc = m.open("a")
    assert m.pages_needed(rc, 9) == [3]
    m.extend(rc, 9)
    assert len(rc.tables[0]) == 3 and rc.length == 0
    m.commit(rc, 9)
    m.extend(rc, 10)                                  # still inside the third page
    assert len(rc.tables[0]) == 3
    m.extend(rc, 13)
    assert len(rc.tables[0]) == 4
    with pytest.raises(ValueError):
        m.commit(rc, 17)                              # beyond its pages
    m.commit(rc, 13)
    other = m.open("b")
    with pytest.raises(PoolExhausted):
        m.extend(other, 17)                           # 5 pages wanted, 4 free
    assert other.tables[0] == [] and m.free_pages() == [4]
    m.close(rc)
    m.close(other)
    with pytest.raises(ValueError):
        m.close(rc)
    m.assert_balanced()


def test_exhaustion_in_one_group_takes_nothing_in_any():
    m = CacheManager({0: KVNeeds(1, 8, None), 1: KVNeeds(1, 8, 64)}, {}, 4, 4, 2, allocate=False)
    rc = m.open("a")
    m.groups[1].pool.allocate(3)                      # someone else holds most of group 1
    with pytest.raises(PoolExhausted):
        m.extend(rc, 8)
    assert rc.tables == [[], []] and m.free_pages() == [4, 1]


def test_window_group_gives_pages_back_as_it_moves():
    m = manager(num_pages=8, page_size=4, window=6)
    rc = m.open("a")
    full, win = 0, 1
    held = []
    for length in range(1, 41):
        m.extend(rc, length)
        m.commit(rc, length)
        first_key = max(0, length - 6 + 1)            # oldest key the next query (position `length`) reads
        assert rc.page_base[win] == first_key // 4
        assert rc.page_base[win] * 4 <= first_key
        assert (rc.page_base[win] + len(rc.tables[win])) * 4 >= length
        held.append(len(rc.tables[win]))
        if length <= 32:
            assert len(rc.tables[full]) == -(-length // 4)
        if length == 32:
            break
    assert max(held) <= 3                             # window 6 over pages of 4: at most 3 pages
    m.close(rc)
    m.assert_balanced()


def test_peak_pages():
    m = manager(num_pages=64, page_size=4, window=6)
    assert m.peak_pages(40, None) == [10, 10]
    assert m.peak_pages(40, 8) == [10, 5]             # window 6 + portion 8 -> 4 pages + 1


def test_random_orders_lose_nothing():
    rng = random.Random(0)
    m = manager(num_pages=24, page_size=4, window=10, slots=5)
    live = {}
    opened = 0
    for _ in range(3000):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            live[opened] = m.open(opened)
            opened += 1
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            rc = live[rid]
            new = rc.length + rng.choice([1, 1, 1, 2, 5, 9])
            if m.can_extend(rc, new):
                m.extend(rc, new)
                m.commit(rc, new)
            else:
                before = [list(t) for t in rc.tables]
                with pytest.raises(PoolExhausted):
                    m.extend(rc, new)
                assert before == rc.tables
        elif live:
            rid = rng.choice(list(live))
            m.close(live.pop(rid))
        for g in m.groups:                            # every page is free or held by exactly one request
            held = [p for rc in live.values() for p in rc.tables[g.index]]
            assert len(held) == len(set(held)) == g.pool.num_live
            assert g.pool.num_live + g.pool.num_free == g.pool.total
        assert len({rc.slot for rc in live.values()}) == len(live) == m.slots.num_live
    for rc in list(live.values()):
        m.close(rc)
    m.assert_balanced()


def test_state_slots_are_zeroed_when_taken_again():
    m = CacheManager({}, {0: StateNeeds((3,))}, 4, 4, 2, dtype=torch.float32, device="cpu")
    a = m.open("a")
    m.state[0][a.slot] += 5
    m.close(a)
    b = m.open("b")
    assert b.slot == a.slot and float(m.state[0][b.slot].abs().sum()) == 0
    with pytest.raises(PoolExhausted):
        m.open("c"), m.open("d")
    assert m.pages_needed(b, 100) == []               # a model without keys and values holds no pages
