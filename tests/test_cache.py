"""The cache's bookkeeping: slots and pages are never lost, held twice or freed
twice; groups with a window give pages back (no GPU: device=None)."""

import random

import pytest
import torch

from reflex_b200 import CacheError, ContextOverflow, InvalidInput, OutOfMemory
from reflex_b200.cache import PAGE_TOKENS, Cache, IdPool, KVSpec, StateSpec


def test_id_pool_take_give():
    p = IdPool(4, "slot")
    a = p.take(3)
    assert sorted(a) == [0, 1, 2] and p.free_count == 1
    with pytest.raises(OutOfMemory):
        p.take(2)
    assert p.free_count == 1  # nothing taken by the failed call
    p.give([1])
    with pytest.raises(CacheError):
        p.give([1])  # freed twice
    with pytest.raises(CacheError):
        p.give([3])  # never taken
    with pytest.raises(CacheError):
        p.give([0, 0])
    assert p.is_held(0) and p.is_held(2) and not p.is_held(1)
    assert p.take(1) == [1]  # a freed id is used again first


def _cache(max_tokens=512, window=None, max_positions=4096, max_slots=None):
    specs = {0: KVSpec(2, 16), 1: KVSpec(2, 16), 2: KVSpec(2, 16, window) if window else KVSpec(2, 16)}
    return Cache(specs, max_tokens, max_positions, torch.float32, None, max_slots=max_slots)


def _invariants(c: Cache):
    for g in c.kv_groups:
        held = []
        for slot in c.lengths:
            held += [int(g.table_host[slot, i]) for i in range(g.first[slot], g.end[slot])]
        assert len(held) == len(set(held)), "a page is held twice"
        assert len(held) == g.pool.held_count, "a page is lost"
        assert all(g.pool.is_held(p) for p in held)
    assert c.slots.held_count == len(c.lengths)


def test_groups_by_need():
    c = _cache(window=40)
    assert len(c.kv_groups) == 2
    assert sorted(len(g.entries) for g in c.kv_groups) == [1, 2]
    c2 = Cache({0: KVSpec(2, 16), 1: StateSpec((4, 3)), 2: None}, 128, 256, torch.float32, None)
    assert len(c2.kv_groups) == 1 and len(c2.state_groups) == 1 and c2.has(2) is None


def test_pages_follow_lengths_and_slots_are_reused():
    c = _cache(max_tokens=512)
    a, b = c.take_slot(), c.take_slot()
    c.reserve([(a, 5), (b, 130)])
    c.commit([(a, 5), (b, 130)])
    g = c.kv_groups[0]
    assert g.end[a] == 1 and g.end[b] == 3
    _invariants(c)
    for _ in range(59):
        c.reserve([(a, 1)])
        c.commit([(a, 1)])
    assert c.length(a) == 64 and g.end[a] == 1
    c.reserve([(a, 1)])
    c.commit([(a, 1)])
    assert g.end[a] == 2
    _invariants(c)
    c.give_slot(a)
    with pytest.raises(CacheError):
        c.give_slot(a)
    with pytest.raises(CacheError):
        c.length(a)
    a2 = c.take_slot()
    assert a2 == a and c.length(a2) == 0
    _invariants(c)
    c.give_slot(b)
    c.give_slot(a2)
    assert all(g.pool.held_count == 0 for g in c.kv_groups)


def test_max_tokens_counts_whole_pages():
    c = _cache(max_tokens=256)  # 4 pages
    s = [c.take_slot() for _ in range(4)]
    c.reserve([(x, 1) for x in s])  # 4 requests of 1 token hold 4 pages
    c.commit([(x, 1) for x in s])
    with pytest.raises(OutOfMemory):
        c.reserve([(s[0], 64)])  # would need a fifth page
    _invariants(c)
    c.give_slot(s[3])
    c.reserve([(s[0], 64)])
    c.commit([(s[0], 64)])
    _invariants(c)
    extra = c.take_slot()  # a slot is free again, but no page is
    with pytest.raises(OutOfMemory):
        c.reserve([(extra, 1)])
    with pytest.raises(OutOfMemory):
        c.take_slot()  # 4 pages -> 4 slots, all held now
    _invariants(c)


def test_reserve_is_all_or_nothing():
    c = _cache(max_tokens=256)
    a, b = c.take_slot(), c.take_slot()
    with pytest.raises(OutOfMemory):
        c.reserve([(a, 100), (b, 200)])
    assert all(g.pool.held_count == 0 for g in c.kv_groups)
    with pytest.raises(InvalidInput):
        c.reserve([(a, 0)])
    _invariants(c)


def test_context_overflow():
    c = _cache(max_tokens=1024, max_positions=100)
    a = c.take_slot()
    with pytest.raises(ContextOverflow) as e:
        c.reserve([(a, 101)])
    assert str(e.value).startswith("context length exceeded")
    c.reserve([(a, 100)])
    c.commit([(a, 100)])
    with pytest.raises(ContextOverflow):
        c.reserve([(a, 1)])


def test_window_group_gives_pages_back():
    c = _cache(max_tokens=2048, window=40)
    wg = next(g for g in c.kv_groups if g.spec.window)
    fg = next(g for g in c.kv_groups if not g.spec.window)
    a = c.take_slot()
    c.reserve([(a, 300)])
    assert wg.pool.held_count == 5  # the whole prompt is needed within its step
    c.commit([(a, 300)])
    # later queries (position >= 300) see keys >= 261: pages 0..3 are dead
    assert wg.first[a] == 4 and wg.pool.held_count == 1 and fg.pool.held_count == 5
    for _ in range(200):
        c.reserve([(a, 1)])
        c.commit([(a, 1)])
        assert wg.pool.held_count <= 2
        _invariants(c)
    c.give_slot(a)
    assert wg.pool.held_count == 0 and fg.pool.held_count == 0


def test_random_traffic_keeps_invariants():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 40, window=70, max_slots=8)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and c.slots.free_count:
            live[c.take_slot()] = 0
        elif op < 0.4 and live:
            s = rng.choice(list(live))
            c.give_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 7, 64, 65, 200])
            try:
                c.reserve([(s, n)])
                c.commit([(s, n)])
                live[s] += n
            except (OutOfMemory, ContextOverflow):
                pass
        _invariants(c)
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.give_slot(s)
    assert all(g.pool.held_count == 0 for g in c.kv_groups) and c.slots.held_count == 0


def test_workspace_regions_take_turns_and_grow_after_the_step():
    """The step's working memory: a request a region cannot hold is served by
    the allocator and remembered; after `settle` the same requests are views
    into the regions, a phase's memory is reused two runs later, what the last
    run made stays untouched, and `keep` memory lives for the whole step."""
    import torch

    from reflex_b200.ops import workspace as wsm

    ws = wsm.Workspace("cpu")

    def one_step():
        made = []
        with wsm.use(ws):
            made.append(wsm.new((10, 8), torch.float32, "cpu", keep=True))
            for run in range(4):
                wsm.next_phase()
                made.append(wsm.new((100,), torch.float32, "cpu"))
                made.append(wsm.new((7, 3), torch.bfloat16, "cpu"))
        ws.settle()
        return made

    one_step()
    assert ws.misses == 9 and ws.nbytes > 0
    a = one_step()
    assert ws.misses == 9  # everything came from the regions this time
    hidden, r0, r1, r2, r3 = a[0], a[1], a[3], a[5], a[7]
    assert r0.data_ptr() == r2.data_ptr() and r1.data_ptr() == r3.data_ptr() and r0.data_ptr() != r1.data_ptr()
    assert all(t.data_ptr() % 256 == 0 for t in a)
    assert hidden.shape == (10, 8) and a[2].dtype == torch.bfloat16
    own = None
    with wsm.use(ws):
        own = wsm.new((5,), torch.float32, "cpu", own=True)
        inside = wsm.new((5,), torch.float32, "cpu")
    bufs = [b for b in ws.buffers() if b is not None]
    lies_in = lambda t: any(b.data_ptr() <= t.data_ptr() < b.data_ptr() + b.numel() for b in bufs)
    assert lies_in(inside) and not lies_in(own)
    assert not lies_in(wsm.new((5,), torch.float32, "cpu"))  # no step: the allocator's
