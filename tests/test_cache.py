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


def test_pool_reference_counts():
    p = PagePool(3)
    a = p.allocate()
    p.retain(a)
    assert p.refcount(a) == 2
    p.release(a)
    assert p.is_held(a) and p.num_free == 2          # one holder is left
    p.release(a)
    assert not p.is_held(a) and p.num_free == 3
    with pytest.raises(InvalidArgument, match="freed twice"):
        p.release(a)
    with pytest.raises(InvalidArgument, match="not held"):
        p.retain(a)
    p.check()


def test_fork_shares_pages_and_a_write_copies_first():
    """A forked request holds its parent's pages; whoever writes into a shared page gets a copy with the same
    content in every member entry, the other keeps the original; full pages stay shared until both are gone."""
    m = CacheManager([FULL, FULL, STATE], 16, 256, 4, 256, device="cpu", dtype=torch.float32)
    g = m.groups[0]
    m.add_request("a")
    m.reserve("a", 40)                                   # blocks 0, 1 full, block 2 half full
    pages_a = m.table_row(g, "a")[:3].tolist()
    for entry in g.members:
        for t, arr in enumerate(g.arrays[entry]):
            for b, p in enumerate(pages_a):
                arr[p] = 100 * entry + 10 * t + b
    m.state_arrays[2][m.slot_of("a")] = 7.0
    free = m.free_pages
    m.fork("a", "b")
    assert m.free_pages == free and m.table_row(g, "b")[:3].tolist() == pages_a
    assert all(g.pool.refcount(p) == 2 for p in pages_a)
    assert torch.all(m.state_arrays[2][m.slot_of("b")] == 7.0) and m.slot_of("b") != m.slot_of("a")
    m.check()
    # b goes on from token 40: block 2 is shared and about to be written -> copied; block 3 is new
    assert m.pages_needed("b", 50, start_pos=40) == 2
    m.reserve("b", 50, write_from=40)
    pages_b = m.table_row(g, "b")[:4].tolist()
    assert pages_b[:2] == pages_a[:2] and pages_b[2] != pages_a[2] and pages_b[3] >= 0
    assert g.pool.refcount(pages_a[2]) == 1 and g.pool.refcount(pages_b[2]) == 1 and g.pool.refcount(pages_a[0]) == 2
    for entry in g.members:
        for t, arr in enumerate(g.arrays[entry]):
            assert torch.all(arr[pages_b[2]] == 100 * entry + 10 * t + 2)     # the copy carries the content
    # a writes too: its block 2 is its own again, nothing is copied
    free = m.free_pages
    m.reserve("a", 41, write_from=40)
    assert m.free_pages == free and m.table_row(g, "a")[:3].tolist() == pages_a
    m.check()
    m.free_request("a")
    assert g.pool.refcount(pages_a[0]) == 1 and g.pool.is_held(pages_a[0]) and not g.pool.is_held(pages_a[2])
    m.free_request("b")
    m.check()
    assert m.free_pages == m.num_pages


def test_copy_on_write_is_all_or_nothing_when_pages_run_out():
    m = manager([FULL], tokens=64, requests=3, context=64)          # 4 pages
    m.add_request("a")
    m.reserve("a", 40)                                              # 3 pages
    m.fork("a", "b")
    m.add_request("c")
    m.reserve("c", 16)                                              # the last page
    before = m.table_row(m.groups[0], "b").copy()
    with pytest.raises(ResourceExhausted):
        m.reserve("b", 41, write_from=40)                           # needs a copy of block 2: no page left
    assert (m.table_row(m.groups[0], "b") == before).all() and m.free_pages == 0
    m.check()


def test_fork_from_fewer_tokens_and_truncate():
    m = manager([FULL, WIN])
    m.add_request("a")
    m.reserve("a", 100)                                             # the parent has reserved ahead of what it computed
    m.fork("a", "b", tokens=70)
    assert m.tokens["b"] == 70 and m.groups[0].tables["b"].length == 5
    m.check()
    assert m.truncate("a", 33) > 0
    assert m.tokens["a"] == 33 and m.groups[0].tables["a"].length == 3
    with pytest.raises(InvalidArgument, match="cannot be cut"):
        m.truncate("a", 34)
    m.reserve("a", 48, write_from=33)                               # block 2 is shared with b: copied
    m.check()
    m.free_request("a")
    m.free_request("b")
    m.check()
    assert m.free_pages == m.num_pages


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_forks(seed):
    """As test_random_orders, with forks and truncations among the operations: every page is counted once per
    table that names it after every operation, and everything is free at the end."""
    rng = random.Random(100 + seed)
    specs = [FULL, WIN, None, FULL] if seed % 2 else [FULL, FULL]
    m = manager(specs, page=16, tokens=rng.choice([96, 160, 512]), requests=6, context=400)
    live = {}
    nxt = 0
    for _ in range(800):
        op = rng.random()
        if op < 0.10 and len(live) < 6:
            m.add_request(nxt)
            live[nxt] = 0
            nxt += 1
        elif op < 0.20 and live and len(live) < 6:
            parent = rng.choice(list(live))
            m.fork(parent, nxt, tokens=live[parent])
            live[nxt] = live[parent]
            nxt += 1
        elif op < 0.27 and live:
            r = rng.choice(list(live))
            # a windowed group has given early pages back: only cut where every group still has its pages
            if all(g.spec.window <= 0 for g in m.groups):
                live[r] = rng.randint(0, live[r])
                m.truncate(r, live[r])
        elif op < 0.88 and live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 16, 33])
            if live[r] + n > 400:
                continue
            free_before = [g.pool.num_free for g in m.groups]
            tables_before = [g.tables[r].pages.copy() for g in m.groups]
            try:
                m.reserve(r, live[r] + n, write_from=live[r])
                for g in m.groups:                     # what it is about to write is its own
                    assert not g.shared_blocks(r, live[r], live[r] + n)
                live[r] += n
                m.advance(r, live[r])
            except ResourceExhausted:
                assert [g.pool.num_free for g in m.groups] == free_before
                assert all((g.tables[r].pages == t).all() for g, t in zip(m.groups, tables_before))
                victim = rng.choice(list(live))
                m.free_request(victim)
                del live[victim]
        elif live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        m.check()
    for r in list(live):
        m.free_request(r)
    m.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in m.groups) and m.free_slots == 6


def test_table_updates_follow_what_changed_not_how_long_requests_are():
    """The device keeps every live request's block table; a step sends only the entries that changed. A request
    with 131,000 tokens that grows by one token costs at most one entry, and nothing at all inside a page."""
    from dynalm_b200.engine.step import _StepBuffers
    spec = CacheSpec("pages", (2, 16))
    window = CacheSpec("pages", (2, 16), window=64)
    m = CacheManager([spec, window], 16, 140000 + 4096, 4, 131072, None, torch.float32)
    m.add_request("long")
    total_updates = 0
    for total in range(1000, 131001, 1000):                  # the prompt comes in portions of 1,000 tokens
        m.reserve("long", total)
        m.advance("long", total)
        ups = m.take_table_updates()
        # all keys: the portion's new blocks; window: the same, and what fell behind the window is given back
        assert len([u for u in ups if u[0] == 0]) <= 64 and len([u for u in ups if u[0] == 1]) <= 64 + 64 + 8
        total_updates += len(ups)
    assert m.take_table_updates() == []
    assert m.groups[1].pool.num_held <= 6                    # the window keeps 64 keys
    sizes = []
    for total in range(131001, 131001 + 40):
        m.reserve("long", total)
        m.advance("long", total)
        ups = m.take_table_updates()
        sizes.append(len(ups))
        slot = m.slot_of("long")
        for gid, s, block, page in ups:
            assert s == slot and (page == -1 or page == int(m.groups[gid].tables["long"].pages[block]))
    assert max(sizes) <= 3 and sum(1 for n in sizes if n == 0) >= 30        # a new page every 16 tokens, per group
    # a second request's entries carry its own slot; freeing forgets what was pending
    m.add_request("b")
    m.reserve("b", 40)
    ups = m.take_table_updates()
    assert {u[1] for u in ups} == {m.slot_of("b")} and len(ups) == 3 + 3
    m.reserve("b", 100)
    m.free_request("b")
    assert m.take_table_updates() == []
    m.check()
    # the step's packed integers do not grow with the context: a few KB for 64 tokens and 4 requests
    small = _StepBuffers("cpu", 64, 4, n_groups=2, max_blocks=131072 // 16, page_size=16, plans=())
    assert small.size * 4 < 16 * 1024
    assert small.tables.shape == (2, 4, 8192)


def test_reserve_that_fails_leaves_windowed_tables_as_they_were():
    spec = CacheSpec("pages", (1, 8), window=32)
    m = CacheManager([spec], 16, 64, 2, 1024, None, torch.float32)
    m.add_request("a")
    m.reserve("a", 20)
    m.advance("a", 20)
    t = m.groups[0].tables["a"]
    before = (t.first, t.length, t.pages.copy())
    m.add_request("b")
    m.reserve("b", 32)                    # the pool is now full (4 pages)
    with pytest.raises(ResourceExhausted):
        m.reserve("a", 700, write_from=600)      # would skip blocks the window has passed, then run out of pages
    assert (t.first, t.length) == before[:2] and (t.pages == before[2]).all()
    m.check()


def test_requests_with_state_cannot_be_cut_back():
    from dynalm_b200.errors import Unsupported
    m = CacheManager([CacheSpec("pages", (1, 8)), CacheSpec("state", state_shape=(4,))], 16, 256, 2, 256, None, torch.float32)
    m.add_request("a")
    m.reserve("a", 40)
    with pytest.raises(Unsupported, match="cannot be rewound"):
        m.truncate("a", 20)
    m.truncate("a", 40)
    m.fork("a", "b", tokens=33)            # reserved but not computed: nothing to rewind
    assert m.tokens["b"] == 33
    m.check()
