"""The cache's bookkeeping (CPU): no slot or page is lost, held twice or freed
twice; groups keep storage of their own; a window gives pages back."""
import random

import pytest
import torch

from mivi_v4_b200.cache import CacheError, IndexPool, KVNeed, KVView, SequenceCache, StateNeed, StateView, plan_cache


def make(n_slots=4, n_pages=8, page=4, needs=None, cache_of=None):
    needs = needs or [StateNeed((2, 8)), KVNeed(2, 8), StateNeed((2, 8)), KVNeed(2, 8)]
    plan = plan_cache(needs, cache_of or [None] * len(needs))
    return SequenceCache(plan, n_slots=n_slots, n_pages=n_pages, page_size=page, dtype=torch.float32, device="cpu")


def test_index_pool_faults():
    p = IndexPool(3, "slot")
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        p.take()
    p.give(b)
    with pytest.raises(CacheError, match="not held"):
        p.give(b)
    with pytest.raises(CacheError, match="outside"):
        p.give(7)
    assert p.take() == b            # a freed index is used again
    p.check()


def test_plan_groups_layers_by_need():
    c = make()
    assert [type(g.need).__name__ for g in c.plan.groups] == ["StateNeed", "KVNeed"]
    assert c.plan.binding == [(0, 0), (1, 0), (0, 1), (1, 1)]
    assert c.storage[0].shape == (2, 4, 2, 8) and c.storage[1].shape == (2, 8, 2, 2, 4, 8)
    # a different head count or a window is another group with storage of its own
    c2 = make(needs=[KVNeed(2, 8), KVNeed(2, 8, window=6), KVNeed(1, 8), None])
    assert len(c2.plan.groups) == 3 and c2.plan.binding[3] is None


def test_plan_shared_cache():
    plan = plan_cache([KVNeed(2, 8), KVNeed(2, 8), KVNeed(2, 8)], [None, 0, None])
    assert plan.binding == [(0, 0), (0, 0), (0, 1)] and plan.owner == [True, False, True]
    with pytest.raises(CacheError, match="not an earlier"):
        plan_cache([KVNeed(2, 8), KVNeed(2, 8)], [1, None])
    with pytest.raises(CacheError, match="keeps"):
        plan_cache([KVNeed(2, 8), KVNeed(1, 8)], [None, 0])


def test_slots_pages_and_lengths():
    c = make()
    s = c.assign()
    assert c.length(s) == 0
    c.reserve(s, 5)
    assert c.pages[1].held_count == 2          # 5 tokens, pages of 4
    c.advance(s, 5)
    c.reserve(s, 1)
    assert c.pages[1].held_count == 2
    c.advance(s, 1)
    c.reserve(s, 3)
    assert c.pages[1].held_count == 3
    assert c.page_rows(1, [s]) == [[0, 1, 2]]
    c.check()
    c.release(s)
    assert c.pages[1].held_count == 0 and c.slots.held_count == 0
    with pytest.raises(CacheError, match="not assigned"):
        c.release(s)
    with pytest.raises(CacheError, match="not assigned"):
        c.length(s)


def test_full_cache_takes_nothing():
    c = make(n_pages=3)
    a, b = c.assign(), c.assign()
    c.reserve(a, 8)
    with pytest.raises(CacheError, match="full"):
        c.reserve(b, 5)
    assert c.pages[1].held_count == 2          # b took no page
    c.reserve(b, 4)
    c.check()


def test_slot_reuse_zeroes_state():
    c = make()
    s = c.assign()
    c.storage[0][:, s] = 7.0
    c.release(s)
    s2 = c.assign()
    assert s2 == s and float(c.storage[0][:, s2].abs().sum()) == 0.0


def test_window_gives_pages_back():
    c = make(needs=[KVNeed(2, 8, window=5)], n_pages=4, page=4)
    s = c.assign()
    total = 0
    for n in [6, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1]:
        c.reserve(s, n)
        c.advance(s, n)
        total += n
        first_needed = max(0, total - 5 + 1)
        pages = c._get(s).pages[0]
        assert all((p is None) == (blk < first_needed // 4) for blk, p in enumerate(pages)), (total, pages)
        c.check()
    assert total == 16 and c.pages[0].held_count <= 2   # 16 tokens never need more than the window's pages
    c.release(s)
    assert c.pages[0].held_count == 0


def test_random_traffic_never_loses_anything():
    rng = random.Random(0)
    c = make(n_slots=5, n_pages=12, page=4)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and c.slots.free_count:
            live[c.assign()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 6)
            try:
                c.reserve(s, n)
                c.advance(s, n)
                live[s] += n
            except CacheError:
                pass
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        c.check()
        assert {s: c.length(s) for s in live} == live
        assert c.pages[1].held_count == sum(-(-n // 4) for n in live.values())
    for s in list(live):
        c.release(s)
    assert c.pages[1].free_count == 12 and c.slots.free_count == 5


def test_grow_slots_keeps_state():
    c = make(n_slots=2)
    a = c.assign()
    c.storage[0][:, a] = 3.0
    c.grow_slots(5)
    assert c.storage[0].shape[1] == 5 and float(c.storage[0][0, a, 0, 0]) == 3.0
    assert sorted(c.assign() for _ in range(4)) == [1, 2, 3, 4]
    c.check()


def test_dump_slot_reads_pages_in_order():
    c = make(n_pages=4, page=4)
    s0 = c.assign()
    s = c.assign()
    c.reserve(s0, 4)
    c.reserve(s, 6)
    c.advance(s, 6)
    pool = c.storage[1]
    for blk, page in enumerate(c._get(s).pages[1]):
        for r in range(4):
            pool[:, page, :, :, r, :] = 10 * blk + r
    d = c.dump_slot(s)[1]
    assert d.shape == (2, 2, 6, 2, 8)
    assert d[0, 0, :, 0, 0].tolist() == [0, 1, 2, 3, 10, 11]


def test_a_position_with_several_needs_gets_several_views():
    """A layer may keep more than one thing: its needs come as a list, each joins the group of its kind
    (shape and dtype included), and the layer gets one view for each, in order."""
    both = [KVNeed(2, 8), StateNeed((3,), torch.bfloat16)]
    plan = plan_cache([StateNeed((3,)), both, None, both, [StateNeed((3,))]], [None, None, None, 1, None])
    assert [g.need for g in plan.groups] == [StateNeed((3,)), KVNeed(2, 8), StateNeed((3,), torch.bfloat16)]
    assert plan.bindings == [[(0, 0)], [(1, 0), (2, 0)], [], [(1, 0), (2, 0)], [(0, 1)]]
    assert plan.several == [False, True, False, True, True] and plan.owner[3] is False
    c = SequenceCache(plan, n_slots=2, n_pages=4, page_size=16, dtype=torch.float32, device="cpu")
    assert c.storage[2].dtype == torch.bfloat16 and c.storage[0].dtype == torch.float32
    tables = {g: torch.zeros(1, 1, dtype=torch.int32) for g in c.kv_groups}
    assert isinstance(c.view(0, tables), StateView) and c.view(2, tables) is None
    kv, st = c.view(1, tables)
    assert isinstance(kv, KVView) and isinstance(st, StateView) and st.state.dtype == torch.bfloat16
    assert [type(v) for v in c.view(4, tables)] == [StateView]
    with pytest.raises(CacheError, match="keeps"):
        plan_cache([both, [KVNeed(2, 8)]], [None, 0])
