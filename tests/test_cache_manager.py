"""The cache manager on the CPU (no tensors): no page lost, held twice or freed twice,
under random orders of requests; groups with different needs; windows; state slots."""
import random

import pytest
import torch

from fastmlx_b200.cache import CacheManager, OutOfPages, PagePool
from fastmlx_b200.parts import PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16)
WIN = PagedKVSpec(2, 16, window=10)
OTHER = PagedKVSpec(1, 32)


def test_pool_is_last_in_first_out_and_guards_double_free():
    p = PagePool(4, 8)
    a = p.take(3)
    assert a == [0, 1, 2] and p.free_pages == 1
    p.give([1])
    assert p.take(1) == [1]                      # the page just given back comes first
    with pytest.raises(OutOfPages):
        p.take(2)
    assert p.free_pages == 1                     # a refused request takes nothing
    p.give([0])
    with pytest.raises(RuntimeError, match="not held"):
        p.give([0])
    with pytest.raises(RuntimeError, match="not held"):
        p.give([7])
    p.check()


def test_layers_with_equal_needs_share_a_group_and_others_get_their_own():
    needs = [(FULL, None, None), (WIN, None, None), (FULL, None, None), (OTHER, None, None), (None, None, 0)]
    m = CacheManager(needs, page_size=4, num_pages=8, max_requests=2, allocate=False)
    assert [g.spec for g in m.groups] == [FULL, WIN, OTHER]
    assert [g.entries for g in m.groups] == [[0, 2], [1], [3]]
    assert [e.group for e in m.entries] == [0, 1, 0, 2, 0]
    assert [e.writable for e in m.entries] == [True, True, True, True, False]


def test_tensors_have_the_documented_layout():
    m = CacheManager([(FULL, StateSpec((3, 5)), None), (FULL, None, None)], page_size=4, num_pages=6, max_requests=2,
                     dtype=torch.float32, device="cpu")
    assert tuple(m.groups[0].kv.shape) == (2, 6, 2, 2, 4, 16)
    assert m.entries[0].kv.data_ptr() == m.groups[0].kv[0].data_ptr()
    assert tuple(m.entries[0].state.shape) == (2, 3, 5) and m.entries[1].state is None
    assert m.bytes_per_token() == 2 * 2 * 2 * 16 * 4


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([(FULL, None, None), (OTHER, None, None)], page_size=4, num_pages=3, max_requests=2, allocate=False)
    a, b = m.add_request("a"), m.add_request("b")
    m.reserve(a, 8)
    m.commit(a)
    with pytest.raises(OutOfPages):
        m.reserve(b, 5)                          # needs 2 pages in each group, 1 is free
    assert b.tables[0].pages == [] and b.tables[1].pages == [] and m.free_pages == 1
    m.check()
    m.reserve(b, 4)
    m.rollback(b)
    assert m.free_pages == 1 and b.length == 0
    m.check()


def test_a_window_gives_pages_back_as_it_passes_them():
    m = CacheManager([(WIN, None, None)], page_size=4, num_pages=16, max_requests=1, allocate=False)
    r = m.add_request("a")
    held = []
    for _ in range(40):
        m.reserve(r, 1)
        m.commit(r)
        m.check()
        bt = r.tables[0]
        first_needed = r.length - 10 + 1          # the next query at position `length` sees keys > length - 10
        for i, p in enumerate(bt.pages):
            if (i + 1) * 4 <= first_needed:
                assert p == -1
            else:
                assert p >= 0
        held.append(len(bt.live()))
    assert max(held) <= 4                          # ceil(10 / 4) + 1 pages at most
    m.free("a")
    assert m.free_pages == 16


def test_a_portion_keeps_the_pages_its_first_token_still_sees():
    m = CacheManager([(WIN, None, None)], page_size=4, num_pages=16, max_requests=1, allocate=False)
    r = m.add_request("a")
    m.reserve(r, 23)
    m.commit(r)                                    # next query at 23 sees keys 14..23: pages 3.. live
    assert r.tables[0].first_live == 3 and r.tables[0].pages[:3] == [-1, -1, -1]


def test_slots_are_zeroed_and_reused():
    m = CacheManager([(FULL, StateSpec((4,)), None)], page_size=4, num_pages=4, max_requests=2, dtype=torch.float32)
    a = m.add_request("a")
    m.entries[0].state[a.slot] += 7
    b = m.add_request("b")
    with pytest.raises(OutOfPages, match="slots"):
        m.add_request("c")
    m.free("a")
    c = m.add_request("c")
    assert c.slot == a.slot and float(m.entries[0].state[c.slot].abs().sum()) == 0.0
    with pytest.raises(KeyError):
        m.add_request("b")
    m.check()


@pytest.mark.parametrize("seed", range(10))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    needs = [(FULL, None, None), (WIN, None, None), (FULL, None, None)]
    m = CacheManager(needs, page_size=rng.choice([2, 4, 16]), num_pages=rng.choice([6, 10, 30]),
                     max_requests=4, allocate=False)
    live = {}
    n_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 4:
            live[n_id] = m.add_request(n_id)
            n_id += 1
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            before = [g.pool.free_pages for g in m.groups]
            try:
                m.reserve(live[rid], rng.choice([1, 1, 1, 2, 5, 17]))
            except OutOfPages:
                assert [g.pool.free_pages for g in m.groups] == before
            else:
                if rng.random() < 0.15:
                    m.rollback(live[rid])
                    assert [g.pool.free_pages for g in m.groups] == before
                else:
                    m.commit(live[rid])
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check()
        for r in live.values():
            need = -(-r.length // m.page_size)
            assert len(r.tables[0].pages) == need and all(p >= 0 for p in r.tables[0].pages)
    m.free_all()
    m.check()
    assert all(g.pool.free_pages == g.pool.num_pages for g in m.groups)
