"""The cache manager: pages with a block table per request, and slots of fixed-size state.

Every run-order entry of a model that keeps a cache declares a `CacheSpec`. Entries whose specs are
equal form a group; a group of kind "pages" has one page pool and, per request, one block table that
is valid for all its member entries at once (as a physical block of the reference is valid in all
layers, dynalm/src/kv_cache/kv_cache.cpp:31-38). Groups with different needs (all keys, a window of
them, another entry shape) have pools and tables of their own. A group with a window gives pages
back as soon as every token in them lies behind the window of the request's next token. Entries of
kind "state" get one row per request slot in an array [slots, *state_shape], zeroed when a slot is
handed out; every request takes a slot whether or not the model has such entries.

What is given back when: all pages and the slot when a request is freed (finished, cancelled,
failed, or preempted for recompute: dynalm/src/runtime/sequence.cpp:44-63); windowed pages after
`advance`; pages past a shorter length after `truncate`.

Requests can share pages: `fork` gives a new request the block tables of a live one (every page
retained once more, as `KvBlockTable::clone`, dynalm/src/kv_cache/kv_cache.cpp:146-151), and
`reserve` copies a shared page before the request writes into it (copy-on-write, as
`make_writable`, kv_cache.cpp:153-168; the copy covers every member entry of the group, as
`copy_block` covers all layers, kv_cache.cpp:77-86). A page goes back to the pool when its last
holder lets go of it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..engine.context import CacheView
from ..errors import InvalidArgument, ResourceExhausted, Unsupported
from ..parts.base import CacheSpec
from .pool import PagePool

DEFAULT_PAGE_SIZE = 16      # tokens per page, the reference's block size (dynalm/src/runtime/engine.cpp:405)


def _torch_dtype(name: Optional[str], default: torch.dtype) -> torch.dtype:
    if name is None:
        return default
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


@dataclass
class _Table:
    pages: np.ndarray            # int32 [max_blocks], -1 = no page
    first: int = 0               # blocks below `first` were given back (window)
    length: int = 0              # blocks [first, length) hold pages
    dirty: List[int] = field(default_factory=list)     # blocks whose page has changed since the device copy was last brought up to date

    def set(self, block: int, page: int) -> None:
        self.pages[block] = page
        self.dirty.append(block)


class PageGroup:
    def __init__(self, gid: int, spec: CacheSpec, page_size: int, num_pages: int, max_blocks: int):
        self.gid = gid
        self.spec = spec
        self.page_size = page_size
        self.pool = PagePool(num_pages)
        self.max_blocks = max_blocks
        self.members: List[int] = []                      # run-order entries
        self.arrays: Dict[int, List[torch.Tensor]] = {}   # entry -> tensors [pages, page_size, *entry_shape]
        self.tables: Dict[Hashable, _Table] = {}
        self.storage: Optional[torch.Tensor] = None

    def first_needed_block(self, next_pos: int) -> int:
        """The lowest block a query at `next_pos` (or later) can still read."""
        if self.spec.window <= 0:
            return 0
        return max(0, next_pos - self.spec.window + 1) // self.page_size

    def shared_blocks(self, req, begin: int, end: int) -> List[int]:
        """Blocks of `req` that hold positions in [begin, end) on pages other requests hold too."""
        t = self.tables.get(req)
        if t is None or end <= begin:
            return []
        lo = max(t.first, begin // self.page_size)
        hi = min(t.length, -(-end // self.page_size))
        return [b for b in range(lo, hi) if t.pages[b] >= 0 and self.pool.refcount(int(t.pages[b])) > 1]

    def blocks_needed(self, req, start_pos: int, total: int) -> int:
        """New pages that holding `total` tokens needs, the next query (and the first position written) being
        at `start_pos`: pages for new blocks, and copies of shared pages the request is about to write into."""
        t = self.tables.get(req)
        have_first, have_len = (t.first, t.length) if t is not None else (0, 0)
        want_len = -(-total // self.page_size)
        lo = max(have_len, self.first_needed_block(start_pos), have_first)
        return max(0, want_len - lo) + len(self.shared_blocks(req, start_pos, total))

    def copy_page(self, src: int, dst: int) -> None:
        """The content of page `src` into page `dst`, for every member entry (layer) of the group."""
        for arrs in self.arrays.values():
            for a in arrs:
                a[dst].copy_(a[src])


class CacheManager:
    """Owns all cache memory of one model.

    specs         per run-order entry, its CacheSpec or None (entries that read another entry's cache
                  and entries without a cache give None)
    max_tokens    tokens all live requests may hold at once; every "pages" group gets
                  ceil(max_tokens / page_size) pages
    max_requests  state slots, and the most requests alive at once
    context       the longest a single request may grow (sets the width of block tables)
    """

    def __init__(self, specs: Sequence[Optional[CacheSpec]], page_size: int, max_tokens: int, max_requests: int,
                 context: int, device, dtype: torch.dtype):
        if page_size <= 0 or max_tokens <= 0 or max_requests <= 0 or context <= 0:
            raise InvalidArgument("cache sizes must be positive")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.context = int(context)
        self.device = torch.device(device) if device is not None else None
        self.dtype = dtype
        self.num_pages = -(-int(max_tokens) // self.page_size)
        self.max_blocks = -(-self.context // self.page_size)
        self.groups: List[PageGroup] = []
        self.entry_group: Dict[int, PageGroup] = {}
        self.state_arrays: Dict[int, torch.Tensor] = {}
        self.state_specs: Dict[int, CacheSpec] = {}
        by_key: Dict[tuple, PageGroup] = {}
        for entry, spec in enumerate(specs):
            if spec is None:
                continue
            if spec.kind == "pages":
                g = by_key.get(spec.group_key())
                if g is None:
                    g = PageGroup(len(self.groups), spec, self.page_size, self.num_pages, self.max_blocks)
                    by_key[spec.group_key()] = g
                    self.groups.append(g)
                g.members.append(entry)
                self.entry_group[entry] = g
            elif spec.kind == "state":
                self.state_specs[entry] = spec
                if self.device is not None:
                    dt = _torch_dtype(spec.dtype, torch.float32)
                    self.state_arrays[entry] = torch.zeros((self.max_requests,) + tuple(spec.state_shape),
                                                           dtype=dt, device=self.device)
            else:
                raise InvalidArgument(f"cache spec of kind '{spec.kind}' is not known (pages, state)")
        if self.device is not None:
            # one allocation per group, [member entries, tensors, pages, page_size, *entry_shape]: every entry's arrays
            # are views of it, and one kernel can clear a page in all of them at once (see take_fresh_pages)
            for g in self.groups:
                dt = _torch_dtype(g.spec.dtype, dtype)
                g.storage = torch.zeros((len(g.members), g.spec.tensors, self.num_pages, self.page_size) + tuple(g.spec.entry_shape),
                                        dtype=dt, device=self.device)
                for i, entry in enumerate(g.members):
                    g.arrays[entry] = [g.storage[i, t] for t in range(g.spec.tensors)]
        self._fresh: List[tuple] = []              # (group id, page) handed out since take_fresh_pages
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))
        self.slots: Dict[Hashable, int] = {}
        self.tokens: Dict[Hashable, int] = {}     # tokens reserved so far per request
        self._dirty: set = set()                  # (group id, request) whose table has changed since take_table_updates

    # ---- requests -----------------------------------------------------------------------------
    def has_request(self, req) -> bool:
        return req in self.slots

    def add_request(self, req) -> int:
        """Take a state slot (zeroed) for a new request; pages come with `reserve`."""
        if req in self.slots:
            raise InvalidArgument(f"request {req!r} is already live")
        if not self._free_slots:
            raise ResourceExhausted("no free request slot")
        slot = self._free_slots.pop()
        self.slots[req] = slot
        self.tokens[req] = 0
        for g in self.groups:
            g.tables[req] = _Table(np.full(g.max_blocks, -1, dtype=np.int32))
        for arr in self.state_arrays.values():
            arr[slot].zero_()
        return slot

    def pages_needed(self, req, total: int, start_pos: Optional[int] = None) -> int:
        """The most pages any group must still allocate so that `req` holds `total` tokens."""
        start = self.tokens.get(req, 0) if start_pos is None else start_pos
        return max((g.blocks_needed(req, start, total) for g in self.groups), default=0)

    def can_reserve(self, req, total: int, headroom: int = 0) -> bool:
        start = self.tokens.get(req, 0)
        return all(g.blocks_needed(req, start, total) + headroom <= g.pool.num_free for g in self.groups)

    def reserve(self, req, total: int, write_from: Optional[int] = None) -> None:
        """Make sure `req` has pages of its own for the positions it is about to write, [write_from, total)
        (`write_from` defaults to the tokens reserved so far), in every group: new pages for new blocks, and a
        private copy of every page in that range that it shares with another request. All or nothing: on
        ResourceExhausted the pages this call took are given back and no table has changed."""
        if req not in self.slots:
            raise InvalidArgument(f"request {req!r} is not live")
        if total > self.context:
            raise InvalidArgument(f"request {req!r} would hold {total} tokens, the context is {self.context}")
        start = self.tokens[req] if write_from is None else min(int(write_from), self.tokens[req])
        taken = []       # (group, table, block, page)
        copies = []      # (group, table, block, shared page, private page)
        moves = []       # (table, first block that gets a page): blocks a window has already passed are never allocated
        try:
            for g in self.groups:
                t = g.tables[req]
                for b in g.shared_blocks(req, start, total):
                    copies.append((g, t, b, int(t.pages[b]), g.pool.allocate()))
            for g in self.groups:
                t = g.tables[req]
                want_len = -(-total // self.page_size)
                lo = max(t.length, g.first_needed_block(start))
                if lo > t.length:
                    moves.append((t, lo))
                for b in range(lo, want_len):
                    taken.append((g, t, b, g.pool.allocate()))
        except ResourceExhausted:
            # nothing has been written into a table yet: give the pages back and leave
            for g, t, b, page in reversed(taken):
                g.pool.release(page)
            for g, t, b, shared, private in copies:
                g.pool.release(private)
            raise
        for t, lo in moves:
            if t.length == t.first:
                t.first = lo
            t.length = lo
        for g, t, b, page in taken:
            t.set(b, page)
            t.length = max(t.length, b + 1)
            self._dirty.add((g.gid, req))
            self._fresh.append((g.gid, page))
        for g, t, b, shared, private in copies:
            g.copy_page(shared, private)
            t.set(b, private)
            g.pool.release(shared)
            self._dirty.add((g.gid, req))
        self.tokens[req] = max(self.tokens[req], total)

    def fork(self, parent, child, tokens: Optional[int] = None) -> int:
        """A new request `child` that holds what `parent` holds: the same pages in every group (each held once
        more; a later write copies first, see `reserve`) and a copy of the parent's state rows in a slot of its
        own. `tokens`: how many of the parent's tokens the child starts from (the parent may have pages reserved
        beyond what it has computed); default all. Returns the child's slot."""
        if parent not in self.slots:
            raise InvalidArgument(f"request {parent!r} is not live")
        slot = self.add_request(child)
        for g in self.groups:
            src, dst = g.tables[parent], g.tables[child]
            dst.pages[:] = src.pages
            dst.first, dst.length = src.first, src.length
            for b in range(src.first, src.length):
                if src.pages[b] >= 0:
                    g.pool.retain(int(src.pages[b]))
                    dst.dirty.append(b)
            self._dirty.add((g.gid, child))
        self.tokens[child] = self.tokens[parent]
        for arr in self.state_arrays.values():
            arr[slot].copy_(arr[self.slots[parent]])
        if tokens is not None and tokens < self.tokens[child]:
            self.truncate(child, tokens, computed_beyond=False)      # the state rows copied above stand at `tokens`
        return slot

    def truncate(self, req, total: int, computed_beyond: bool = True) -> int:
        """`req` keeps its first `total` tokens only: pages wholly past them are given back
        (`KvBlockTable::truncate`, dynalm/src/kv_cache/kv_cache.cpp:137-144). Returns the pages let go.
        `computed_beyond` False says that nothing past `total` has been computed yet (pages were only reserved), so
        that per-request state has nothing to take back."""
        if req not in self.slots:
            raise InvalidArgument(f"request {req!r} is not live")
        if total < 0 or total > self.tokens[req]:
            raise InvalidArgument(f"request {req!r} holds {self.tokens[req]} tokens, it cannot be cut to {total}")
        if self.state_specs and computed_beyond and total < self.tokens[req]:
            # state of fixed size has no history to go back to: such a request is recomputed, not cut
            raise Unsupported(f"request {req!r} cannot be cut back: the model keeps per-request state that cannot be rewound")
        n = 0
        keep = -(-total // self.page_size)
        for g in self.groups:
            t = g.tables[req]
            for b in range(max(keep, t.first), t.length):
                if t.pages[b] >= 0:
                    g.pool.release(int(t.pages[b]))
                    t.set(b, -1)
                    self._dirty.add((g.gid, req))
                    n += 1
            t.length = max(min(t.length, keep), min(t.first, keep))
            t.first = min(t.first, t.length)
        self.tokens[req] = total
        return n

    def advance(self, req, computed: int) -> int:
        """`req` has now computed `computed` tokens; give back pages that every window has passed.
        Returns the number of pages given back."""
        n = 0
        for g in self.groups:
            if g.spec.window <= 0:
                continue
            t = g.tables[req]
            keep_from = min(g.first_needed_block(computed), t.length)
            for b in range(t.first, keep_from):
                if t.pages[b] >= 0:
                    g.pool.release(int(t.pages[b]))
                    t.set(b, -1)
                    self._dirty.add((g.gid, req))
                    n += 1
            t.first = max(t.first, keep_from)
        return n

    def free_request(self, req) -> None:
        """Give back every page and the slot of `req`."""
        slot = self.slots.pop(req, None)
        if slot is None:
            raise InvalidArgument(f"request {req!r} is not live (freed twice?)")
        for g in self.groups:
            t = g.tables.pop(req)
            for b in range(t.first, t.length):
                if t.pages[b] >= 0:
                    g.pool.release(int(t.pages[b]))
            self._dirty.discard((g.gid, req))
        self.tokens.pop(req)
        self._free_slots.append(slot)

    # ---- what the step function reads ---------------------------------------------------------------
    def slot_of(self, req) -> int:
        return self.slots[req]

    def table_row(self, group: PageGroup, req) -> np.ndarray:
        return group.tables[req].pages

    def take_fresh_pages(self) -> List[tuple]:
        """(group id, page) of every page handed out since the last call. A page keeps what its previous owner wrote;
        the step function clears these before the step that first writes into them, so that the slots of a request's
        last page beyond its newest token never hold another request's values (a kernel that copies whole pages
        multiplies them by a probability of zero, and zero times a stray infinity is not zero)."""
        out, self._fresh = self._fresh, []
        return out

    def take_table_updates(self) -> List[tuple]:
        """What has changed in the block tables since the last call, as (group id, slot, block, page): the device
        keeps a copy of every live request's table in the row of its slot, and a step brings it up to date with
        these alone, so a step's cost on the host and on the bus follows what changed, not how long the requests
        are. A page of -1 marks a block that was given back."""
        out = []
        for gid, req in sorted(self._dirty, key=lambda k: (k[0], self.slots[k[1]])):
            t = self.groups[gid].tables[req]
            slot = self.slots[req]
            seen = set()
            for b in reversed(t.dirty):            # the last change of a block wins
                if b not in seen:
                    seen.add(b)
                    out.append((gid, slot, b, int(t.pages[b])))
            t.dirty.clear()
        self._dirty.clear()
        return out

    def view(self, entry: int, block_tables: Dict[int, torch.Tensor]) -> Optional[CacheView]:
        g = self.entry_group.get(entry)
        if g is not None:
            return CacheView("pages", g.arrays[entry], self.page_size, block_tables[g.gid])
        if entry in self.state_arrays:
            return CacheView("state", [self.state_arrays[entry]])
        return None

    # ---- accounting -----------------------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=self.num_pages)

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def bytes(self) -> int:
        n = 0
        for g in self.groups:
            for arrs in g.arrays.values():
                n += sum(a.numel() * a.element_size() for a in arrs)
        n += sum(a.numel() * a.element_size() for a in self.state_arrays.values())
        return n

    def check(self) -> None:
        """No page lost or freed twice, every page counted once per table that names it; no slot held twice."""
        for g in self.groups:
            g.pool.check()
            holders: Dict[int, int] = {}
            for req, t in g.tables.items():
                for b in range(g.max_blocks):
                    p = int(t.pages[b])
                    inside = t.first <= b < t.length
                    if p >= 0:
                        if not inside:
                            raise AssertionError(f"request {req!r} keeps page {p} outside its table range")
                        if not g.pool.is_held(p):
                            raise AssertionError(f"page {p} of {req!r} is on the free list")
                        holders[p] = holders.get(p, 0) + 1
                    elif inside and g.spec.window <= 0:
                        raise AssertionError(f"request {req!r} lacks a page for block {b}")
            for p, n in holders.items():
                if g.pool.refcount(p) != n:
                    raise AssertionError(f"page {p} is named by {n} tables but counted {g.pool.refcount(p)} times")
            if len(holders) != g.pool.num_held:
                raise AssertionError(f"{g.pool.num_held} pages are held but tables name {len(holders)}")
        used = sorted(self.slots.values())
        if len(set(used)) != len(used) or set(used) & set(self._free_slots):
            raise AssertionError("a state slot is held twice")
        if len(used) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot is lost")
