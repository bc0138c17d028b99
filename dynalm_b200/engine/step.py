"""The step function: run one batch of (request, its next tokens) from the cache.

Contract (the reference's `Transformer::forward_batch`, dynalm/src/model/transformer.h:55-75,
preconditions at transformer.cpp:502-535): a step holds any number of requests, each a run of
consecutive positions continuing where that request stopped: a portion of a prompt, or one decoded
token. Portions sit beside single tokens in one batch. The step runs only the tokens it is given,
writes their keys and values into the cache as a side effect, and returns float32 logits for the
wanted rows only, in batch order.
"""

from __future__ import annotations

from dataclasses import dataclass
import os
import time
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..errors import InvalidArgument
from .context import StepContext
from .model import Decoder
from .runtime import Runtime


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places among them (0-based) whose
    logits are wanted."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


SMALL_STEP_ROWS = 256      # steps of up to this many rows use the small set of step buffers


class StepShape:
    """What a step looks like on the host, for the parts' step plans: per entry of the batch its number of rows,
    first row, first position and request slot."""

    __slots__ = ("q_len", "q_start", "pos_start", "slots", "num_tokens")

    def __init__(self, q_len, q_start, pos_start, slots, num_tokens):
        self.q_len, self.q_start, self.pos_start, self.slots, self.num_tokens = q_len, q_start, pos_start, slots, num_tokens


class _StepBuffers:
    """Per-step integers, packed: one pinned host array per ring slot, one device array with fixed
    addresses (kernels captured in a CUDA graph keep reading the same pointers). A step fills a host
    slot and issues one host-to-device copy; a slot is reused only after its copy has completed.

    Beside the step's own arrays it has a section for every step plan a part asked for (`plans`: objects with
    `name`, `ints(max_tokens, max_requests)` and `fill(host_section, shape) -> meta`), and one for the changes of
    the block tables. The block tables themselves stay on the device: `tables` [groups, request slots, blocks per
    request], one row per slot, brought up to date by the step that changes them."""

    RING = 4

    def __init__(self, device, max_tokens: int, max_requests: int, n_groups: int, max_blocks: int, page_size: int,
                 plans=(), tables: Optional[torch.Tensor] = None):
        self.max_tokens, self.max_requests = max_tokens, max_requests
        off = 0
        self.off: Dict[str, slice] = {}

        def take(name, n):
            nonlocal off
            self.off[name] = slice(off, off + n)
            off += (n + 3) // 4 * 4       # 16-byte aligned sections

        for name in ("token_ids", "positions", "row_request", "row_slot", "logit_rows"):
            take(name, max_tokens)
        take("q_start", max_requests + 1)
        for name in ("pos_start", "kv_len", "state_slots", "feedback_src"):
            take(name, max_requests)
        self.plans = list(plans)
        for plan in self.plans:
            take(f"plan:{plan.name}", int(plan.ints(max_tokens, max_requests)))
        # changed table entries of one step: new pages of the tokens it brings, pages windows gave back, a few copies
        self.max_updates = max(1, n_groups) * (max_tokens // max(1, page_size) + 4 * max_requests) + 64
        take("table_updates", 4 * self.max_updates)
        self.max_fresh = self.max_updates
        take("fresh_pages", 2 * self.max_fresh)
        self.size = off
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        self.host = [torch.zeros(self.size, dtype=torch.int32) for _ in range(self.RING)]
        if on_gpu:
            self.host = [h.pin_memory() for h in self.host]
        self.host_np = [h.numpy() for h in self.host]
        self.events = [None] * self.RING
        self.dev = torch.zeros(self.size, dtype=torch.int32, device=self.device)
        self.tables = tables if tables is not None else torch.full((max(1, n_groups), max_requests, max_blocks), -1,
                                                                  dtype=torch.int32, device=self.device)
        self.turn = 0
        self.views = {name: self.dev[sl] for name, sl in self.off.items()}

    def next_host(self) -> int:
        i = self.turn
        self.turn = (self.turn + 1) % self.RING
        if self.events[i] is not None:
            self.events[i].synchronize()
        return i

    def upload(self, i: int, section: Optional[str] = None) -> None:
        """The whole of host slot i, or one section of it, to the device (in stream order)."""
        if section is None:
            self.dev.copy_(self.host[i], non_blocking=True)
        else:
            sec = self.off[section]
            self.dev[sec].copy_(self.host[i][sec], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev

    def dev_view(self, name: str) -> torch.Tensor:
        return self.dev[self.off[name]]


class BatchBuilder:
    """Turns a list of entries into a StepContext: checks it, reserves pages, flattens it into the
    packed buffers and uploads them. It also keeps, per live request, how many tokens are in the cache."""

    def __init__(self, cache: CacheManager, runtime: Runtime, max_requests: int, vocab: int, plans=()):
        self.cache = cache
        self.rt = runtime
        self.max_tokens = runtime.max_tokens
        self.max_requests = int(max_requests)
        self.vocab = int(vocab)
        names = set()
        plans = [p for p in plans if not (p.name in names or names.add(p.name))]
        self.buffers = _StepBuffers(runtime.device, self.max_tokens, self.max_requests, len(cache.groups),
                                    cache.max_blocks, cache.page_size, plans)
        # steps of few rows (every decode step) have buffers of their own, a few KB instead of five arrays of
        # max_tokens entries: what crosses the bus follows the step, and the addresses a CUDA graph holds stay fixed
        self.small = (_StepBuffers(runtime.device, SMALL_STEP_ROWS, self.max_requests, len(cache.groups), cache.max_blocks,
                                   cache.page_size, plans, tables=self.buffers.tables)
                      if self.max_tokens > SMALL_STEP_ROWS else self.buffers)
        self.computed: Dict[Hashable, int] = {}       # tokens each live request has in the cache
        self.tables = {g.gid: self.buffers.tables[g.gid] for g in cache.groups}      # [request slots, blocks]
        self.update_launches = 0
        self.last_upload_bytes = 0

    def begin(self, request) -> None:
        self.cache.add_request(request)
        self.computed[request] = 0

    def end(self, request) -> None:
        self.cache.free_request(request)
        del self.computed[request]

    def fork(self, parent, child) -> None:
        """`child` starts as a copy of `parent`: it shares the parent's pages (copied when either writes into one)
        and goes on from the parent's computed tokens."""
        if parent not in self.computed:
            raise InvalidArgument(f"request {parent!r} is not live")
        self.cache.fork(parent, child, tokens=self.computed[parent])
        self.computed[child] = self.computed[parent]

    def _reserve_all(self, entries: Sequence[StepEntry]) -> None:
        """Pages for every entry's tokens, or nothing: when one entry cannot get its pages, the requests this call
        began are ended again and the others give back what this call reserved for them."""
        begun, grown = [], []
        try:
            for e in entries:
                if e.request not in self.computed:
                    self.begin(e.request)
                    begun.append(e.request)
                else:
                    grown.append((e.request, self.cache.tokens[e.request]))
                self.cache.reserve(e.request, self.computed[e.request] + len(e.tokens), write_from=self.computed[e.request])
        except Exception:
            for req in begun:
                self.end(req)
            for req, before in grown:
                if self.cache.tokens[req] > before:
                    self.cache.truncate(req, before, computed_beyond=False)
            raise

    def _table_updates(self, b: _StepBuffers, h, slot: int) -> int:
        """Write what has changed in the block tables into the step's section (and send whatever does not fit in
        rounds of its own first). Returns the number of entries that travel with the step."""
        ups = self.cache.take_table_updates()
        sec = b.off["table_updates"]
        while len(ups) > b.max_updates:
            head, ups = ups[:b.max_updates], ups[b.max_updates:]
            h[sec][:4 * len(head)] = np.asarray(head, dtype=np.int32).reshape(-1)
            b.upload(slot, "table_updates")
            self._apply(b, len(head))
            if b.events[slot] is not None:
                b.events[slot].synchronize()       # the section is written again right away
        if ups:
            h[sec][:4 * len(ups)] = np.asarray(ups, dtype=np.int32).reshape(-1)
        return len(ups)

    def _clear(self, b: _StepBuffers, h, slot: int, fresh, upload: bool) -> None:
        """Pages that were just handed out are set to zero in every array of their group, before the step writes."""
        from ..kernels import ops
        if upload:
            h[b.off["fresh_pages"]][:2 * len(fresh)] = np.asarray(fresh, dtype=np.int32).reshape(-1)
            b.upload(slot, "fresh_pages")
        for gid in sorted({g for g, _ in fresh}):
            ops.zero_pages(self.cache.groups[gid].storage, b.views["fresh_pages"], len(fresh), gid)
        if upload and b.events[slot] is not None:
            b.events[slot].synchronize()

    def _apply(self, b: _StepBuffers, n: int) -> None:
        from ..kernels import ops
        ops.table_updates(b.tables, b.views["table_updates"], n)
        self.update_launches += 1

    def build(self, entries: Sequence[StepEntry], reserve: bool = True,
              feedback_src: Optional[Sequence[int]] = None) -> StepContext:
        """Check the batch, reserve pages (unless the caller already has), flatten it and upload it.
        `feedback_src[r]` (one-token entries only): the place in the previous step's chosen ids that row r's
        token comes from on the device, or -1 to keep the token given here."""
        if not entries:
            raise InvalidArgument("a step needs at least one entry")
        if len(entries) > self.max_requests:
            raise InvalidArgument(f"{len(entries)} requests in one step, the engine was made for {self.max_requests}")
        total = sum(len(e.tokens) for e in entries)
        if total > self.max_tokens:
            raise InvalidArgument(f"{total} tokens in one step, the engine was made for {self.max_tokens}")
        seen = set()
        for e in entries:
            if len(e.tokens) == 0:
                raise InvalidArgument(f"request {e.request!r} brings no tokens")
            if e.request in seen:
                raise InvalidArgument(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise InvalidArgument(f"request {e.request!r} wants place {w} of {len(e.tokens)} tokens")
            if min(e.tokens) < 0 or max(e.tokens) >= self.vocab:
                raise InvalidArgument(f"request {e.request!r} has a token id outside [0, {self.vocab})")
        if reserve:
            self._reserve_all(entries)
        else:
            for e in entries:
                if e.request not in self.computed:
                    raise InvalidArgument(f"request {e.request!r} is not live")
                if self.cache.tokens[e.request] < self.computed[e.request] + len(e.tokens):
                    raise InvalidArgument(f"request {e.request!r} has no pages reserved for its tokens")

        b = self.small if total <= self.small.max_tokens else self.buffers
        i = b.next_host()
        h = b.host_np[i]
        off = b.off
        tok = h[off["token_ids"]]
        pos = h[off["positions"]]
        rreq = h[off["row_request"]]
        rslot = h[off["row_slot"]]
        lrows = h[off["logit_rows"]]
        q_start = h[off["q_start"]]
        pos_start = h[off["pos_start"]]
        kv_len = h[off["kv_len"]]
        slots = h[off["state_slots"]]
        r0 = 0
        n_logit = 0
        h_q_len, h_q_start, h_pos_start, h_slots = [], [], [], []
        for r, e in enumerate(entries):
            n = len(e.tokens)
            start = self.computed[e.request]
            slot = self.cache.slot_of(e.request)
            tok[r0:r0 + n] = e.tokens
            pos[r0:r0 + n] = np.arange(start, start + n, dtype=np.int32)
            rreq[r0:r0 + n] = r
            rslot[r0:r0 + n] = slot
            for w in e.want:
                lrows[n_logit] = r0 + w
                n_logit += 1
            q_start[r] = r0
            pos_start[r] = start
            kv_len[r] = start + n
            slots[r] = slot
            h_q_len.append(n)
            h_q_start.append(r0)
            h_pos_start.append(start)
            h_slots.append(slot)
            r0 += n
        q_start[len(entries)] = r0
        shape = StepShape(h_q_len, h_q_start, h_pos_start, h_slots, total)
        extras = {}
        for plan in b.plans:
            extras[plan.name] = (b.views[f"plan:{plan.name}"], plan.fill(h[off[f"plan:{plan.name}"]], shape))
        if feedback_src is not None:
            if total != len(entries) or len(feedback_src) != len(entries):
                raise InvalidArgument("token feedback needs one token per entry and one source per entry")
            h[off["feedback_src"]][:len(entries)] = feedback_src
        n_updates = self._table_updates(b, h, i)
        fresh = self.cache.take_fresh_pages()
        while len(fresh) > b.max_fresh:             # (more than a step's section holds: in rounds of their own)
            head, fresh = fresh[:b.max_fresh], fresh[b.max_fresh:]
            self._clear(b, h, i, head, upload=True)
        if fresh:
            h[off["fresh_pages"]][:2 * len(fresh)] = np.asarray(fresh, dtype=np.int32).reshape(-1)
        b.upload(i)
        self.last_upload_bytes = b.size * 4
        if n_updates:
            self._apply(b, n_updates)
        if fresh:
            self._clear(b, h, i, fresh, upload=False)
        d = b.views
        extras["step:feedback_src"] = d["feedback_src"]
        return StepContext(
            num_tokens=total, num_requests=len(entries), token_ids=d["token_ids"], positions=d["positions"],
            row_request=d["row_request"], row_slot=d["row_slot"], q_start=d["q_start"], pos_start=d["pos_start"],
            kv_len=d["kv_len"], state_slots=d["state_slots"], logit_rows=d["logit_rows"], num_logit_rows=n_logit,
            h_q_len=h_q_len, h_pos_start=h_pos_start, h_state_slots=h_slots, block_tables=self.tables,
            decode_only=all(n == 1 for n in h_q_len), max_q_len=max(h_q_len),
            max_kv_len=max(s + n for s, n in zip(h_pos_start, h_q_len)), extras=extras)

    def finish(self, entries: Sequence[StepEntry]) -> None:
        """The step has been issued: count its tokens and let windows give pages back."""
        for e in entries:
            self.computed[e.request] += len(e.tokens)
            self.cache.advance(e.request, self.computed[e.request])


class StepFunction:
    """Model + cache + the step. `step(entries)` is the whole forward path; generation, the
    scheduler and trace replay all go through it."""

    def __init__(self, model: Decoder, cache: CacheManager, runtime: Runtime, max_requests: int,
                 use_graphs: bool = True):
        self.model = model
        self.cache = cache
        self.rt = runtime
        self.max_tokens = runtime.max_tokens
        self.max_requests = int(max_requests)
        self.vocab = model.vocab
        self.batcher = BatchBuilder(cache, runtime, max_requests, model.vocab, model.step_plans())
        self.buffers = self.batcher.buffers
        self.computed = self.batcher.computed
        self._logits: Optional[torch.Tensor] = None
        self._caches = None
        # Decode-only steps (one token per request) are captured once per (requests, wanted rows,
        # span bucket) as a CUDA graph and replayed: the kernels read the step's integers from the
        # packed device buffer, whose addresses never change. The reference's GPU path keeps one
        # prepared graph per step structure in the same way, at most 64 of them
        # (dynacore/include/dynacore/gpu/ggml_device.h:8-13,39-48).
        from ..kernels import ops as _ops
        self.use_graphs = bool(use_graphs) and model.graph_safe and not _ops.CHECKED     # a checked build reads a record after every launch
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._decode_logits: Optional[torch.Tensor] = None
        self.graph_kernel_launches = 0     # kernels replayed through graphs so far
        self._graph_nodes: Dict[tuple, int] = {}
        self._captured_logits: Dict[tuple, bool] = {}     # whether a captured step leaves logits (or only chosen ids)
        self._shape_seen: Dict[tuple, int] = {}     # decode-only launch shape -> how often it has come
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self.graph_captures = 0            # graphs captured so far, and the host time that took
        self.graph_capture_ms = 0.0

    # ---- request lifetime ----------------------------------------------------------------------
    def begin(self, request) -> None:
        self.batcher.begin(request)

    def end(self, request) -> None:
        """The request is finished (or dropped for recompute): its pages and slot are given back."""
        self.batcher.end(request)

    def fork(self, parent, child) -> None:
        """A new request that continues from where `parent` stands now, sharing the parent's cache pages; whichever
        of the two writes into a shared page first gets a copy of it (the reference's fork and copy-on-write,
        dynalm/src/kv_cache/kv_cache.cpp:146-168)."""
        self.batcher.fork(parent, child)

    def live(self) -> List[Hashable]:
        return list(self.computed)

    # ---- the step ----------------------------------------------------------------------------------
    def _logits_buffer(self, rows: int) -> torch.Tensor:
        if self._logits is None or self._logits.shape[0] < rows:
            cap = 1 << (max(rows, 8) - 1).bit_length()
            self._logits = None
            self._logits = torch.empty((min(cap, max(self.max_tokens, rows)), self.vocab), dtype=torch.float32,
                                       device=self.rt.device)
        return self._logits

    def caches(self):
        if self._caches is None:
            self._caches = [self.cache.view(i, self.batcher.tables) for i in range(len(self.model.order))]
        return self._caches

    def step(self, entries: Sequence[StepEntry], reserve: bool = True, token_feedback=None,
             choose=None) -> Optional[torch.Tensor]:
        """Run the batch. Returns float32 logits [wanted rows, vocab] on the device (a view of a
        buffer that the next step overwrites), or None when nothing was wanted.

        token_feedback = (chosen ids on the device, [source place per entry]): the tokens of this step's
        one-token entries are taken on the device from the ids a previous step chose, so the step can be
        issued before those ids have reached the host.

        choose = (ids, status_to), int32 tensors on the device: the caller wants nothing but the most likely token of
        every wanted row, in ids[0 .. wanted rows). Where the head can pick it in its product's epilogue the logits are
        never written and None is returned; else the logits are returned as without `choose` and the caller picks."""
        if token_feedback is None:
            ctx = self.batcher.build(entries, reserve)
        else:
            from ..kernels import ops
            chosen, src = token_feedback
            ctx = self.batcher.build(entries, reserve, feedback_src=src)
            ops.feedback_tokens(ctx.token_ids, chosen, ctx.extras["step:feedback_src"], len(entries))
        if self.use_graphs and ctx.decode_only:
            logits = self._replay(ctx, choose)
        else:
            out = self._logits_buffer(ctx.num_logit_rows) if ctx.num_logit_rows else None
            logits = self._forward(ctx, out, choose)
        self.batcher.finish(entries)
        return logits

    def _capture(self, key: tuple, ctx: StepContext, out: Optional[torch.Tensor], choose=None) -> torch.cuda.CUDAGraph:
        """The step's launches as a CUDA graph (nothing runs yet). Captured on a stream of its own between
        capture_begin and capture_end, without the collection of garbage and the emptying of the allocator's
        cache that torch's context manager does first: nothing is allocated in here."""
        from ..kernels import ops
        started = time.perf_counter()
        if len(self._graphs) >= self.MAX_GRAPHS:
            old = next(iter(self._graphs))
            del self._graphs[old]
            self._graph_nodes.pop(old, None)
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.rt.device)
        graph = torch.cuda.CUDAGraph()
        current = torch.cuda.current_stream()
        self._capture_stream.wait_stream(current)
        before = ops.LAUNCHES
        with torch.cuda.stream(self._capture_stream):
            graph.capture_begin()
            try:
                self._captured_logits[key] = self._forward(ctx, out, choose) is not None
            finally:
                graph.capture_end()
        current.wait_stream(self._capture_stream)
        self._graph_nodes[key] = ops.LAUNCHES - before
        self._graphs[key] = graph
        self.graph_captures += 1
        self.graph_capture_ms += (time.perf_counter() - started) * 1e3
        return graph

    def _forward(self, ctx: StepContext, out: Optional[torch.Tensor], choose=None) -> Optional[torch.Tensor]:
        from ..kernels import ops
        with ops.pinned_stream():
            return self.model.forward(ctx, self.caches(), out, choose)

    MAX_GRAPHS = 64
    # A launch shape is captured when it comes for the eighth time. A capture costs 5 to 15 ms on the host; shapes
    # that pass by (the last requests of a batch ending one after the other: 64, 63, 62, ... rows for two steps
    # each) are cheaper run as they are, and the plain runs before a capture have allocated every workspace and
    # loaded every kernel that the capture will meet. Measured on continuous batching (3B shape, 32 requests):
    # 2.20 s with a capture at first sight (32 captures), 2.05 s at the third time (26), 2.04 s at the eighth (2).
    GRAPH_AFTER = int(os.environ.get("DYNALM_GRAPH_AFTER", "8"))

    def _replay(self, ctx: StepContext, choose=None) -> Optional[torch.Tensor]:
        if self._decode_logits is None:
            self._decode_logits = torch.empty((self.max_requests, self.vocab), dtype=torch.float32,
                                              device=self.rt.device)
        # a graph holds the addresses it was captured with: the tensors of `choose` are part of its key
        chosen = None if choose is None else tuple(None if t is None else t.data_ptr() for t in choose)
        key = (ctx.num_requests, ctx.num_logit_rows, chosen) + self.model.graph_key(ctx)
        out = self._decode_logits if ctx.num_logit_rows else None
        graph = self._graphs.get(key)
        if graph is None:
            seen = self._shape_seen.get(key, 0) + 1
            self._shape_seen[key] = seen
            if seen < self.GRAPH_AFTER:
                got = self._forward(ctx, out, choose)
                return got[:ctx.num_logit_rows] if got is not None else None
            graph = self._capture(key, ctx, out, choose)
        graph.replay()
        self.graph_kernel_launches += self._graph_nodes[key]
        return out[:ctx.num_logit_rows] if (out is not None and self._captured_logits[key]) else None
