"""The cache manager's accounting without a GPU: no page lost, held twice or freed twice, under
random orders of requests; pages are used again; a window gives pages back as it passes them."""

import random

import pytest
import torch

from omniserver_b200.cache import CacheManager, OutOfPages, OutOfSlots, PagePool, StateSlots
from omniserver_b200.models.decoder import EntryNeeds
from omniserver_b200.parts.base import KVCacheNeed, StateNeed


def manager(num_pages=16, page_size=4, windows=(None, None, 6, 6), max_requests=4, cache_of=None):
    needs = [EntryNeeds(KVCacheNeed(2, 8, w), [], None) for w in windows]
    if cache_of is not None:
        needs.append(EntryNeeds(KVCacheNeed(2, 8, windows[cache_of]), [], cache_of))
    shared = [StateNeed("rope_cursor", (2,), torch.int32, shared=True)]
    return CacheManager(needs, shared, page_size, num_pages, max_requests, torch.float32, "cpu", allocate=False)


def test_page_pool_refuses_double_free_and_reuses_last_freed():
    p = PagePool(3)
    a, b = p.alloc(), p.alloc()
    p.free(a)
    with pytest.raises(ValueError, match="freed twice"):
        p.free(a)
    assert p.alloc() == a            # last freed, first reused
    c = p.alloc()
    with pytest.raises(OutOfPages):
        p.alloc()
    for x in (a, b, c):
        p.free(x)
    assert p.num_free == 3


def test_state_slots_zeroed_on_alloc_and_bounded():
    s = StateSlots(2, {"acc": ((3,), torch.float32)}, "cpu")
    a = s.alloc()
    s.write("acc", a, [1.0, 2.0, 3.0])
    s.free(a)
    b = s.alloc()
    assert b == a and not s.tensors["acc"][b].any()
    s.alloc()
    with pytest.raises(OutOfSlots):
        s.alloc()
    with pytest.raises(ValueError):
        s.free(5)


def test_groups_follow_the_layers_needs():
    m = manager(cache_of=0)
    assert [g.window for g in m.groups] == [None, 6]
    assert [g.entries for g in m.groups] == [[0, 1], [2, 3]]
    b = m.bindings()
    assert [x.group for x in b] == [0, 0, 1, 1, 0]
    assert [x.writes for x in b] == [True, True, True, True, False]


def test_reserve_commit_finish_and_window_release():
    m = manager()
    m.begin("a")
    assert m.pages_needed("a", 10) == [3, 3]
    m.reserve("a", 10)
    assert m.block_table(0, ["a"]).shape == (1, 3)
    sm = m.slot_map(0, ["a"], [10])
    bt = m.block_table(0, ["a"])[0]
    assert list(sm[:4]) == [bt[0] * 4 + i for i in range(4)] and sm[9] == bt[2] * 4 + 1
    m.commit("a", 10)
    # window 6 at cursor 10: future queries see keys >= 5 -> page 0 (keys 0..3) is given back
    assert m.requests["a"].tables[1][0] == -1 and m.requests["a"].tables[1][1] >= 0
    assert m.pages_in_use() == [3, 2]
    m.check_invariants()
    m.reserve("a", 1)
    m.commit("a", 1)
    m.reserve("a", 9)          # a portion longer than the window still gets every page it writes
    assert m.pages_in_use() == [5, 4]
    m.commit("a", 9)           # cursor 20: keys >= 15 -> pages 0..2 gone
    assert m.requests["a"].tables[1][:3] == [-1, -1, -1] and m.pages_in_use() == [5, 2]
    m.finish("a")
    assert m.pages_in_use() == [0, 0] and m.state.num_free == 4


def test_reserve_is_all_or_nothing():
    m = manager(num_pages=4)
    m.begin("a")
    m.begin("b")
    m.reserve("a", 12)
    assert not m.can_reserve([("b", 8)])
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert m.pages_in_use() == [3, 3] and m.requests["b"].tables == [[], []]
    assert m.can_reserve([("b", 4)])


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_double_hold_a_page(seed):
    rng = random.Random(seed)
    m = manager(num_pages=24, page_size=4, max_requests=5)
    live, n_started, reused = {}, 0, False
    seen_pages = set()
    for _ in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            rid = f"r{n_started}"
            n_started += 1
            m.begin(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 16])
            if m.can_reserve([(rid, n)]):
                m.reserve(rid, n)
                for g in range(2):
                    for p in m.requests[rid].tables[g]:
                        if p >= 0:
                            reused |= (g, p) in seen_pages and False
                m.commit(rid, n)
                live[rid] += n
                assert m.requests[rid].cursor == live[rid]
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            (m.reset if rng.random() < 0.2 else m.finish)(rid)
            if rid in m.requests:
                live[rid] = 0
            else:
                del live[rid]
        m.check_invariants()
        for gi, g in enumerate(m.groups):
            assert g.pool.num_free + g.pool.num_held == 24
    for rid in list(live):
        m.finish(rid)
    assert m.pages_in_use() == [0, 0] and m.state.num_free == 5
    with pytest.raises(KeyError):
        m.finish("r0")


def test_a_borrowed_cache_must_match():
    needs = [EntryNeeds(KVCacheNeed(2, 8, None), [], None), EntryNeeds(KVCacheNeed(4, 8, None), [], 0)]
    with pytest.raises(ValueError, match="cannot read the cache"):
        CacheManager(needs, [], 4, 4, 2, torch.float32, "cpu", allocate=False)
