"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back early; state slots; failed reservations change nothing."""
import random

import pytest

from marin_b200.cache import DROPPED, CacheManager, OutOfPages, PageAccountingError, PagePool
from marin_b200.parts import PagedKV, StateNeed


def test_page_pool_accounting():
    pool = PagePool(5)
    a = pool.alloc(3)
    assert len(set(a)) == 3 and pool.num_free == 2 and pool.num_held == 3
    with pytest.raises(OutOfPages):
        pool.alloc(3)
    assert pool.num_free == 2                        # a failed allocation takes nothing
    pool.free(a[:2])
    with pytest.raises(PageAccountingError):
        pool.free([a[0]])                            # freed twice
    with pytest.raises(PageAccountingError):
        pool.free([99])                              # never held
    b = pool.alloc(2)
    assert set(b) == set(a[:2])                      # pages given back are handed out again (LIFO)
    pool.check()


def manager(num_pages=12, window=None, page=4, extra_group=False, state=False, max_requests=4):
    needs = [PagedKV(2, 16, None), PagedKV(2, 16, None), PagedKV(2, 16, window) if window else PagedKV(2, 16, None)]
    cache_of = [None, None, None]
    if extra_group:
        needs.append(PagedKV(1, 32, None))
        cache_of.append(None)
    if state:
        needs.append(StateNeed((8,)))
        cache_of.append(None)
    needs.append(None)          # an entry that reads entry 0's cache
    cache_of.append(0)
    return CacheManager(needs, cache_of, page, num_pages, max_requests)


def test_groups_are_formed_by_need():
    m = manager(window=10, extra_group=True, state=True)
    assert [g.need.window for g in m.groups] == [None, 10, None]
    assert [g.entries for g in m.groups] == [[0, 1], [2], [3]]
    assert m.place[1] == (0, 1) and list(m.state_needs) == [4]


def test_reserve_commit_release():
    m = manager(num_pages=5)
    m.admit("a")
    m.reserve("a", 9)                                   # 3 pages of 4
    assert m.block_table("a", 0) and len(m.block_table("a", 0)) == 3 and m.free_pages() == [2]
    m.commit("a", 9)
    m.reserve("a", 10)                                  # still inside the third page
    assert m.free_pages() == [2]
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 13)                              # 4 pages wanted, 2 free
    assert m.free_pages() == [2] and m.block_table("b", 0) == []
    assert not m.can_reserve([("a", 16), ("b", 8)]) and m.can_reserve([("a", 12), ("b", 8)])
    m.check()
    m.release("a")
    m.reserve("b", 13)
    m.check()
    m.release("b")
    assert m.free_pages() == [5] and m.slots.num_held == 0
    with pytest.raises(KeyError):
        m.release("b")


def test_window_gives_pages_back_when_it_has_passed_them():
    m = manager(num_pages=8, window=6)
    m.admit("a")
    held = []
    for length in range(1, 33):
        m.reserve("a", length)
        m.commit("a", length)
        table = m.block_table("a", 1)
        live = [p for p in table if p != DROPPED]
        held.append(len(live))
        # the next query sits at `length`; it reads keys length-5 .. length: their pages must be there
        for key in range(max(0, length - 6 + 1), length):
            assert table[key // 4] != DROPPED
        m.check()
    assert max(held) <= 3 and len(m.block_table("a", 0)) == 8       # the windowed group stays small, the full one grows
    assert m.groups[1].pool.num_held <= 3
    m.release("a")
    assert m.free_pages() == [8, 8]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = manager(num_pages=rng.choice([6, 9, 20]), window=rng.choice([None, 5, 9]), extra_group=seed % 2 == 0, state=True)
    lengths = {}
    for step in range(600):
        op = rng.random()
        if op < 0.25 and len(lengths) < 4:
            rid = f"r{step}"
            m.admit(rid)
            lengths[rid] = 0
        elif op < 0.8 and lengths:
            rid = rng.choice(list(lengths))
            new_len = lengths[rid] + rng.choice([1, 1, 1, 2, 5, 11])
            before = (m.free_pages(), [list(p) for p in m.requests[rid].pages])
            try:
                m.reserve(rid, new_len)
            except OutOfPages:
                assert (m.free_pages(), [list(p) for p in m.requests[rid].pages]) == before
            else:
                if rng.random() < 0.9:
                    m.commit(rid, new_len)
                    lengths[rid] = new_len
        elif lengths:
            rid = rng.choice(list(lengths))
            m.release(rid)
            del lengths[rid]
        m.check()
    for rid in list(lengths):
        m.release(rid)
    m.check()
    assert all(g.pool.num_held == 0 for g in m.groups) and m.slots.num_held == 0


def test_state_slots():
    m = manager(state=True, max_requests=2)
    a, b = m.admit("a"), m.admit("b")
    assert a.slot != b.slot
    with pytest.raises(OutOfPages):
        m.admit("c")                                    # no slot left
    assert "c" not in m.requests
    m.release("a")
    assert m.admit("c").slot == a.slot                  # the slot is used again
    with pytest.raises(KeyError):
        m.admit("c")
    m.check()
