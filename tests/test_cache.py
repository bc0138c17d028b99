"""The cache manager on the CPU: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; groups keep pages of their own; state slots."""

import random

import pytest
import torch

from dynalm_b200.cache import CacheManager, PagePool
from dynalm_b200.errors import InvalidArgument, ResourceExhausted
from dynalm_b200.parts.base import CacheSpec

FULL = CacheSpec("pages", entry_shape=(2, 16), tensors=2, window=0)
WIN = CacheSpec("pages", entry_shape=(2, 16), tensors=2, window=40)
STATE = CacheSpec("state", state_shape=(4, 8))


def manager(specs, page=16, tokens=256, requests=4, context=256):
    return CacheManager(specs, page, tokens, requests, context, device=None, dtype=torch.float32)


def test_pool_order_and_double_free():
    p = PagePool(4)
    assert [p.allocate() for _ in range(4)] == [0, 1, 2, 3]          # lowest ids first
    with pytest.raises(ResourceExhausted, match="KV cache is full"):
        p.allocate()
    p.release(2)
    p.release(0)
    assert p.allocate() == 0 and p.allocate() == 2                   # the last freed comes first
    p.release(1)
    with pytest.raises(InvalidArgument, match="freed twice"):
        p.release(1)
    with pytest.raises(InvalidArgument):
        p.release(9)
    p.check()


def test_reserve_free_reuse():
    m = manager([FULL, FULL, None])
    assert len(m.groups) == 1 and m.groups[0].members == [0, 1] and m.num_pages == 16
    m.add_request("a")
    m.reserve("a", 17)
    assert m.groups[0].tables["a"].length == 2 and m.free_pages == 14
    m.reserve("a", 17)                                                   # idempotent
    m.reserve("a", 32)
    assert m.free_pages == 14
    m.reserve("a", 33)
    assert m.free_pages == 13
    first_pages = m.table_row(m.groups[0], "a")[:3].tolist()
    m.free_request("a")
    assert m.free_pages == 16
    with pytest.raises(InvalidArgument, match="not live"):
        m.free_request("a")
    m.add_request("b")
    m.reserve("b", 48)
    assert sorted(m.table_row(m.groups[0], "b")[:3].tolist()) == sorted(first_pages)   # the same pages again
    m.check()


def test_exhaustion_is_all_or_nothing():
    m = manager([FULL], tokens=64, context=256)
    m.add_request("a")
    m.add_request("b")
    m.reserve("a", 40)                      # 3 of 4 pages
    with pytest.raises(ResourceExhausted):
        m.reserve("b", 33)                  # needs 3, one is free
    assert m.free_pages == 1 and m.groups[0].tables["b"].length == 0
    m.check()
    assert not m.can_reserve("b", 33) and m.can_reserve("b", 16) and not m.can_reserve("b", 16, headroom=1)
    with pytest.raises(InvalidArgument, match="context"):
        m.reserve("a", 257)


def test_groups_have_pages_of_their_own_and_windows_give_back():
    m = manager([FULL, WIN, FULL, WIN], tokens=256)
    assert len(m.groups) == 2
    full, win = m.groups
    assert full.members == [0, 2] and win.members == [1, 3]
    m.add_request("a")
    pos = 0
    for n in (16, 7, 2, 50, 1, 1, 1, 30, 1):
        m.reserve("a", pos + n)
        pos += n
        m.advance("a", pos)
        m.check()
        t = win.tables["a"]
        # every block a later query can read is there; every block wholly behind the window is not
        lo_block = max(0, pos - 40 + 1) // 16
        assert t.first == lo_block
        assert all(t.pages[b] >= 0 for b in range(lo_block, -(-pos // 16)))
        assert all(t.pages[b] < 0 for b in range(lo_block))
    assert full.pool.num_held == -(-pos // 16)
    assert win.pool.num_held <= 40 // 16 + 2
    m.free_request("a")
    assert full.pool.num_free == win.pool.num_free == m.num_pages
    m.check()


def test_state_slots():
    m = manager([FULL, STATE], requests=2)
    assert set(m.state_specs) == {1}
    s0 = m.add_request("a")
    s1 = m.add_request("b")
    assert {s0, s1} == {0, 1}
    with pytest.raises(ResourceExhausted, match="slot"):
        m.add_request("c")
    with pytest.raises(InvalidArgument, match="already live"):
        m.add_request("a")
    m.free_request("a")
    assert m.add_request("c") == s0
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders(seed):
    """Requests come, grow by random portions, finish or are dropped in random order; after every
    operation no page is lost, held twice or freed twice, and at the end everything is free."""
    rng = random.Random(seed)
    specs = [FULL, WIN, None, FULL] if seed % 2 else [FULL, FULL]
    m = manager(specs, page=16, tokens=rng.choice([96, 160, 512]), requests=5, context=400)
    live = {}
    nxt = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 5:
            m.add_request(nxt)
            live[nxt] = 0
            nxt += 1
        elif op < 0.85 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 16, 33])
            if live[r] + n > 400:
                continue
            free_before = [g.pool.num_free for g in m.groups]
            try:
                m.reserve(r, live[r] + n)
                live[r] += n
                m.advance(r, live[r])
            except ResourceExhausted:
                assert [g.pool.num_free for g in m.groups] == free_before
                victim = rng.choice(list(live))                  # a preemption: drop someone
                m.free_request(victim)
                del live[victim]
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        m.check()
        for g in m.groups:
            held = sum(int((t.pages >= 0).sum()) for t in g.tables.values())
            assert held + g.pool.num_free == g.pool.num_pages
    for r in list(live):
        m.free_request(r)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups) and m.free_slots == 5
