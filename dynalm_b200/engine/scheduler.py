"""Continuous batching above the step function.

One iteration (`Scheduler.step`): take in new requests, retire finished ones, admit waiting ones
while pages allow, plan a batch under the token budgets (decode rows first, then prompt portions),
run it, sample where a request's pending work was completed, emit events. The decisions follow the
reference's scheduler (dynalm/src/scheduler/scheduler.cpp:234-353 admission and validation,
:357-378 preemption, :380-778 the step; sequence states dynalm/src/runtime/sequence.cpp:24-93).

Decoding one step ahead: when the executor can `launch` a batch and `collect` it later (the GPU executor can,
for decode batches sampled on the device), a decode batch is issued without waiting for its tokens, and the
next call of `step` issues the following decode batch BEFORE collecting the first: the new batch takes its
tokens on the device from what the previous one chose. The host's work for a step then overlaps the GPU's, and
the events of a batch are returned one call later. This happens only in the steady state (nothing incoming or
waiting, no cancellation, every running request in that batch); a request that ends on a stop token has one
surplus token computed, whose result is dropped; a request that ends by length is never issued past its end.

When pages run out while a batch is planned, the most recently admitted OTHER running request is
preempted: all its pages are given back, it keeps its generated tokens, goes to the front of the
waiting queue and is recomputed (prompt and generated tokens as one prompt) when it is admitted
again. If nothing can be preempted the request fails with "request needs more KV than the cache
holds". A request whose prompt plus max_new_tokens cannot fit the pool even alone is refused when
it is taken in.

The scheduler drives an `Executor`: something with a cache manager and a `run(batch)` that
computes the batch and returns the sampled token of every item that asked for one. The GPU
executor is `dynalm_b200.engine.executor.GpuExecutor`; tests use a fake to check decisions on the CPU.
"""

from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Protocol, Sequence

from ..cache import CacheManager
from ..errors import EngineError, InvalidArgument, ResourceExhausted
from ..sampling import Sampler, SamplingParams

WAITING, PREFILL, DECODE, FINISHED, CANCELLED, ERROR = "waiting", "prefill", "decode", "finished", "cancelled", "error"
FINISH_EOG, FINISH_LENGTH, FINISH_STOPPED = "eog", "length", "stopped"


@dataclass
class SchedulerConfig:
    """Budgets per step, in tokens. The defaults are the reference's GPU profile
    (dynalm/src/runtime/engine.h:131,152-153; dynalm/src/scheduler/scheduler.h:130-137)."""

    max_running: int = 64
    decode_token_budget: int = 64
    prefill_token_budget: int = 256
    max_prefill_chunk: int = 128          # per request per step; 0 = up to the budget
    max_batch_tokens: int = 512
    context_length: int = 1 << 24         # prompt + max_new_tokens may not exceed it
    # Decode-protected prefill (dynalm/src/scheduler/scheduler.h:138-150): in steps that also carry decode rows the
    # prompt rows are capped by a budget that halves (down to protected_prefill_min) after a mixed step that took
    # longer than decode_latency_target x the recent decode-only step time, and doubles (up to prefill_token_budget)
    # after one that took less than half of that. Steps without decode rows keep the full budget.
    decode_protect: bool = True
    protected_prefill_min: int = 32
    decode_latency_target: float = 6.0
    # Solo prefill (dynalm/src/scheduler/scheduler.h:165-187, scheduler.cpp:436-472): a step without decode rows in
    # which exactly one request is prefilling gives it portions of solo_prefill_chunk rows under a budget of at least
    # that many, instead of max_prefill_chunk and prefill_token_budget: fewer, larger products for a lone prompt.
    # With several prompts prefilling the step is as ever, unless solo_prefill_split shares the solo budget among
    # them (each up to max(max_prefill_chunk, solo_prefill_chunk / prompts)). 0 = off.
    solo_prefill_chunk: int = 0
    solo_prefill_split: bool = False

    def clamp(self) -> None:
        # both budgets must fit one forward pass (scheduler.cpp:91-96)
        self.decode_token_budget = max(1, min(self.decode_token_budget, self.max_batch_tokens - 1))
        self.prefill_token_budget = max(1, min(self.prefill_token_budget,
                                               self.max_batch_tokens - self.decode_token_budget))
        self.solo_prefill_chunk = max(0, min(self.solo_prefill_chunk, self.max_batch_tokens))


@dataclass
class Request:
    """What a caller submits."""

    prompt: Sequence[int]
    max_new_tokens: int = 128
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_token_ids: Sequence[int] = ()     # end-of-generation ids; generation stops after one is sampled
    priority: int = 0
    timeout_ms: float = 0.0                # > 0: the request fails once it has been in the scheduler this long
    on_event: Optional[Callable[["Event"], None]] = None


@dataclass
class Event:
    request_id: int
    token: Optional[int]             # the token sampled in this step, None on a bare final event
    finished: bool = False
    status: str = DECODE
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0


class SequenceState:
    """A request in flight: its tokens, how many are in the cache, its state
    (dynalm/src/runtime/sequence.h:40-101)."""

    def __init__(self, rid: int, req: Request, arrival: int):
        self.id = rid
        self.req = req
        self.tokens: List[int] = list(req.prompt)
        self.prompt_len = len(self.tokens)
        self.num_computed = 0
        self.status = WAITING
        self.finish_reason: Optional[str] = None
        self.error: Optional[str] = None
        self.preemptions = 0
        self.arrival = arrival
        self.admit_order = 0
        self.last_step = 0
        self.sampler: Optional[Sampler] = None      # made once the request has passed validation
        self.cancel_requested = False
        self.deadline: float = 0.0                  # on the scheduler's clock; 0 = none
        self.trace: Optional["RequestTrace"] = None  # filled along the way when the scheduler keeps traces

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.num_computed

    @property
    def generated(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def terminal(self) -> bool:
        return self.status in (FINISHED, CANCELLED, ERROR)

    def mark_computed(self, n: int) -> None:
        self.num_computed += n
        self.status = PREFILL if self.num_computed < self.prompt_len else DECODE

    def append_token(self, tok: int) -> None:
        self.tokens.append(tok)
        if tok in self.req.stop_token_ids:
            self.status, self.finish_reason = FINISHED, FINISH_EOG
        elif self.generated >= self.req.max_new_tokens:
            self.status, self.finish_reason = FINISHED, FINISH_LENGTH


@dataclass
class BatchItem:
    seq: SequenceState
    start: int
    tokens: List[int]
    sample: bool                     # this portion completes the pending work: sample its last row


class Executor(Protocol):
    cache: CacheManager
    max_tokens: int

    def begin(self, request_id: Hashable) -> None: ...
    def end(self, request_id: Hashable) -> None: ...
    def run(self, batch: List[BatchItem]) -> Dict[Hashable, int]: ...


@dataclass
class StepTrace:
    """What one step computed (dynalm/src/scheduler/scheduler.h:98-125)."""

    step: int
    decode_rows: int
    prefill_rows: int
    items: List[tuple]               # (request id, start, n, sampled)
    preempted: List[int]
    admitted: List[int]
    free_pages_after: int


@dataclass
class RequestTrace:
    """One request's life, kept when it ends if the scheduler keeps traces (dynalm/src/scheduler/scheduler.h:113-125).
    Times are on the scheduler's clock, in seconds; 0 = never happened."""

    id: int
    prompt_tokens: int
    generated: int = 0
    submit_s: float = 0.0
    admit_s: float = 0.0
    first_scheduled_s: float = 0.0
    first_token_s: float = 0.0
    finish_s: float = 0.0
    prefill_steps: int = 0               # steps in which it computed prompt rows (again after a preemption)
    prefill_forward_ms: float = 0.0      # forward time of those steps
    preemptions: int = 0
    status: str = WAITING


@dataclass
class SchedulerStats:
    steps: int = 0
    steps_decode_only: int = 0
    steps_prefill_only: int = 0
    steps_mixed: int = 0
    steps_solo_prefill: int = 0           # steps in which a lone prompt got the solo chunk
    admitted: int = 0
    finished: int = 0
    failed: int = 0
    preemptions: int = 0
    tokens_prefilled: int = 0
    tokens_decoded: int = 0
    forward_decode_only_ms: float = 0.0
    forward_prefill_only_ms: float = 0.0
    forward_mixed_ms: float = 0.0
    timed_out: int = 0
    plan_ms: float = 0.0                  # host time spent choosing batches and reserving their pages
    emit_ms: float = 0.0                  # host time spent in the requests' callbacks
    mixed_prefill_budget: int = 0         # the prompt rows a step with decode rows may carry now


class Scheduler:
    def __init__(self, executor: Executor, config: SchedulerConfig = None, keep_trace: bool = False,
                 clock: Callable[[], float] = time.monotonic):
        self.ex = executor
        self.clock = clock                 # seconds; deadlines are measured on it
        self.cfg = config or SchedulerConfig()
        self.cfg.max_batch_tokens = min(self.cfg.max_batch_tokens, executor.max_tokens)
        self.cfg.max_running = min(self.cfg.max_running, executor.cache.max_requests)
        self.cfg.clamp()
        self.incoming: List[SequenceState] = []
        self.waiting: Deque[SequenceState] = deque()
        self.running: List[SequenceState] = []
        self.by_id: Dict[int, SequenceState] = {}
        self.stats = SchedulerStats()
        self.trace: Optional[List[StepTrace]] = [] if keep_trace else None
        self.request_traces: Optional[List[RequestTrace]] = [] if keep_trace else None      # in the order they end
        self._last_forward_ms = 0.0
        self._next_id = 1
        self._arrivals = 0
        self._admit_counter = 0
        self._callbacks: Dict[int, Callable[[Event], None]] = {}
        self._last_rows = (0, 0)
        self._inflight = None          # (batch, what executor.launch returned, launch time): issued, not yet collected
        self._last_done = 0.0
        self._decode_step_ema_ms = 0.0     # recent decode-only step time (0.8 old + 0.2 new, scheduler.cpp:601)
        self._mixed_prefill_budget = self.cfg.prefill_token_budget
        self.stats.mixed_prefill_budget = self._mixed_prefill_budget
        self.lookahead = hasattr(executor, "launch") and hasattr(executor, "collect")
        # `submit` and `cancel` may come from any thread (scheduler.cpp:167-190): they only touch what this lock
        # guards (the hand-off list, the cancel list, the id counter, the table of callbacks); `step` takes both
        # lists over at its top and everything else belongs to the thread that calls `step`.
        self._handoff = threading.Lock()
        self._cancels: List[int] = []
        self.on_submit: Optional[Callable[[], None]] = None      # called after every submit and cancel (an engine's wake-up)

    # ---- submission ----------------------------------------------------------------------------------
    def submit(self, req: Request) -> int:
        """Thread-safe. The request is taken in at the top of the next `step`; an invalid one fails through its
        callback then."""
        with self._handoff:
            rid = self._next_id
            self._next_id += 1
            self._arrivals += 1
            seq = SequenceState(rid, req, self._arrivals)
            if req.timeout_ms > 0:
                seq.deadline = self.clock() + req.timeout_ms / 1000.0
            if self.request_traces is not None:
                seq.trace = RequestTrace(rid, seq.prompt_len, submit_s=self.clock())
            self.incoming.append(seq)
            if req.on_event is not None:
                self._callbacks[rid] = req.on_event
        if self.on_submit is not None:
            self.on_submit()
        return rid

    def cancel(self, rid: int) -> None:
        """Thread-safe; takes effect at the next `step`. Unknown ids are ignored."""
        with self._handoff:
            self._cancels.append(rid)
        if self.on_submit is not None:
            self.on_submit()

    def cancel_all(self) -> None:
        """Thread-safe: every request known at the next `step` is cancelled."""
        self.cancel(None)

    @property
    def idle(self) -> bool:
        with self._handoff:
            return not (self.incoming or self._cancels or self.waiting or self.running or self._inflight)

    def _take_handoff(self) -> List[SequenceState]:
        """What other threads have handed over since the last step: new requests (returned) and cancellations (marked)."""
        with self._handoff:
            new, self.incoming = self.incoming, []
            cancels, self._cancels = self._cancels, []
        for seq in new:
            self.by_id[seq.id] = seq
        for rid in cancels:
            for seq in (list(self.by_id.values()) if rid is None else [self.by_id.get(rid)]):
                if seq is not None:
                    seq.cancel_requested = True
        return new

    # ---- one iteration ---------------------------------------------------------------------------------
    def _fail(self, seq: SequenceState, msg: str, events: List[Event]) -> None:
        seq.status, seq.error = ERROR, msg
        self.stats.failed += 1
        events.append(self._final_event(seq, None))

    def _final_event(self, seq: SequenceState, token: Optional[int]) -> Event:
        if seq.trace is not None and self.request_traces is not None:
            t = seq.trace
            t.generated, t.preemptions, t.status, t.finish_s = seq.generated, seq.preemptions, seq.status, self.clock()
            self.request_traces.append(t)
            seq.trace = None
        return Event(seq.id, token, True, seq.status, seq.finish_reason, seq.error, seq.prompt_len, seq.generated)

    def _drain_incoming(self, events: List[Event]) -> None:
        """Validate new requests (scheduler.cpp:245-275) and queue them by priority, then arrival."""
        cache = self.ex.cache
        vocab = getattr(self.ex, "vocab", None)
        incoming = self._take_handoff()
        for seq in incoming:
            req = seq.req
            try:
                req.sampling.validate()
                if len(req.prompt) == 0:
                    raise InvalidArgument("empty prompt")
                if req.max_new_tokens <= 0:
                    raise InvalidArgument("max_new_tokens must be > 0")
                total = len(req.prompt) + req.max_new_tokens
                if total > self.cfg.context_length:
                    raise InvalidArgument(f"prompt ({len(req.prompt)}) + max_new_tokens ({req.max_new_tokens}) "
                                          f"exceeds the context length {self.cfg.context_length}")
                if total > cache.context or -(-total // cache.page_size) > cache.num_pages:
                    raise InvalidArgument("request could never fit the KV cache even alone")
                if vocab is not None and (min(req.prompt) < 0 or max(req.prompt) >= vocab):
                    raise InvalidArgument(f"token id outside [0, {vocab})")
            except EngineError as e:
                self._fail(seq, str(e), events)
                self.by_id.pop(seq.id, None)
                continue
            seq.sampler = Sampler(req.sampling)
            self.waiting.append(seq)
        if incoming:
            self.waiting = deque(sorted(self.waiting, key=lambda s: (-s.req.priority, s.arrival)))

    def _expire_deadlines(self, events: List[Event]) -> None:
        """Requests past their deadline fail (dynalm/src/scheduler/scheduler.cpp:293-309): running ones are retired
        with the others of this step, waiting ones leave the queue here."""
        now = self.clock()
        for seq in self.running:
            if not seq.terminal and seq.deadline and now > seq.deadline:
                seq.status, seq.error = ERROR, "request timed out"
                self.stats.failed += 1
                self.stats.timed_out += 1
                events.append(self._final_event(seq, None))
        if any(seq.deadline and now > seq.deadline for seq in self.waiting):
            keep = deque()
            for seq in self.waiting:
                if seq.deadline and now > seq.deadline:
                    self._fail(seq, "request timed out while queued", events)
                    self.stats.timed_out += 1
                    self.by_id.pop(seq.id, None)
                else:
                    keep.append(seq)
            self.waiting = keep

    def _retire(self, events: List[Event]) -> None:
        keep = []
        for seq in self.running:
            if seq.cancel_requested and not seq.terminal:
                seq.status = CANCELLED
                events.append(self._final_event(seq, None))
            if seq.terminal:
                self.ex.end(seq.id)
                self.by_id.pop(seq.id, None)
            else:
                keep.append(seq)
        self.running = keep
        for seq in [s for s in self.waiting if s.cancel_requested]:
            self.waiting.remove(seq)
            seq.status = CANCELLED
            self.by_id.pop(seq.id, None)
            events.append(self._final_event(seq, None))

    def _admit(self, admitted: List[int]) -> None:
        """While there is room: the pending tokens plus one page of headroom must fit now
        (scheduler.cpp:311-353)."""
        cache = self.ex.cache
        promised = 0        # pages of requests admitted in this pass, which reserve only when planned
        while self.waiting and len(self.running) < self.cfg.max_running:
            seq = self.waiting[0]
            need = -(-seq.pending // cache.page_size) + 1
            if cache.free_pages - promised < need and self.running:
                break
            if cache.free_slots == 0:
                break
            self.waiting.popleft()
            promised += need - 1
            self.ex.begin(seq.id)
            self._admit_counter += 1
            seq.admit_order = self._admit_counter
            if seq.preemptions == 0:
                self.stats.admitted += 1
                if seq.trace is not None:
                    seq.trace.admit_s = self.clock()
            seq.status = PREFILL
            self.running.append(seq)
            admitted.append(seq.id)

    def _preempt_one(self, keep: SequenceState, preempted: List[int]) -> bool:
        """Give back all pages of the most recently admitted running request other than `keep`
        and send it to the front of the waiting queue for recomputation (scheduler.cpp:357-378)."""
        victim = None
        for s in self.running:
            if s is keep or s.terminal or self.ex.cache.tokens.get(s.id, 0) == 0:
                continue
            if victim is None or s.admit_order > victim.admit_order:
                victim = s
        if victim is None:
            return False
        self.ex.end(victim.id)
        victim.num_computed = 0
        victim.status = WAITING
        victim.preemptions += 1
        self.stats.preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)
        preempted.append(victim.id)
        return True

    def _plan(self, events: List[Event], preempted: List[int]) -> List[BatchItem]:
        cfg, cache = self.cfg, self.ex.cache
        for attempt in range(65):
            batch: List[BatchItem] = []
            decode_rows = prefill_rows = 0
            restart = False

            def is_decode(s: SequenceState) -> bool:
                return s.status == DECODE and s.pending == 1

            order = sorted((s for s in self.running if not s.terminal and s.pending > 0),
                           key=lambda s: (0, s.last_step, s.admit_order) if is_decode(s)
                           else (1, -s.req.priority, s.admit_order))
            # beside decode rows the prompt rows are capped by the adaptive budget
            any_decode = any(is_decode(s) for s in order)
            prefill_budget = (min(cfg.prefill_token_budget, self._mixed_prefill_budget)
                              if cfg.decode_protect and any_decode else cfg.prefill_token_budget)
            prefill_chunk = cfg.max_prefill_chunk
            prefilling = sum(1 for s in order if not is_decode(s))
            solo = (cfg.solo_prefill_chunk > 0 and not any_decode and prefilling > 0
                    and (prefilling == 1 or cfg.solo_prefill_split))
            if solo:
                prefill_budget = max(cfg.prefill_token_budget, cfg.solo_prefill_chunk)
                prefill_chunk = cfg.solo_prefill_chunk
                if prefilling > 1:
                    prefill_chunk = max(cfg.max_prefill_chunk, cfg.solo_prefill_chunk // prefilling, 1)
            for seq in order:
                decode = is_decode(seq)
                used = decode_rows if decode else prefill_rows
                budget = cfg.decode_token_budget if decode else prefill_budget
                n = min(seq.pending, budget - used)
                if not decode and prefill_chunk > 0:
                    n = min(n, prefill_chunk)
                if n <= 0:
                    continue
                try:
                    cache.reserve(seq.id, seq.num_computed + n, write_from=seq.num_computed)
                except ResourceExhausted:
                    if attempt < 64 and self._preempt_one(seq, preempted):
                        restart = True
                        break
                    self._fail(seq, "request needs more KV than the cache holds", events)
                    continue
                start = seq.num_computed
                batch.append(BatchItem(seq, start, seq.tokens[start:start + n], sample=(n == seq.pending)))
                if decode:
                    decode_rows += n
                else:
                    prefill_rows += n
            if not restart:
                self._last_rows = (decode_rows, prefill_rows)
                if solo and prefill_rows > 0:
                    self.stats.steps_solo_prefill += 1
                return batch
        return []

    def _plan_ahead(self, prev: List[BatchItem]) -> Optional[List[BatchItem]]:
        """The decode batch that follows `prev` (issued, not yet collected), or None when the steady state does
        not hold. Tokens are placeholders: the executor feeds them on the device from what `prev` chose."""
        if self.incoming or self._cancels or self.waiting or len(prev) != len(self.running):
            return None
        if any(s.cancel_requested or s.terminal for s in self.running):
            return None
        if any(s.deadline for s in self.running) and any(s.deadline and self.clock() > s.deadline for s in self.running):
            return None
        if sum(1 for b in prev if b.seq.generated + 1 < b.seq.req.max_new_tokens) > self.cfg.decode_token_budget:
            return None
        nxt: List[BatchItem] = []
        try:
            for b in prev:
                seq = b.seq
                if seq.generated + 1 >= seq.req.max_new_tokens:
                    continue                                  # `prev` gives it its last token
                start = b.start + len(b.tokens)
                self.ex.cache.reserve(seq.id, start + 1, write_from=start)
                nxt.append(BatchItem(seq, start, [0], sample=True))
        except ResourceExhausted:
            return None                                       # the ordinary path will preempt
        return nxt or None

    def _dispatch(self, events: List[Event]) -> List[Event]:
        if self._callbacks and events:
            t0 = time.perf_counter()
            for ev in events:
                with self._handoff:
                    seq_cb = self._callbacks.pop(ev.request_id, None) if ev.finished else self._callbacks.get(ev.request_id)
                if seq_cb is not None:
                    seq_cb(ev)
            self.stats.emit_ms += (time.perf_counter() - t0) * 1e3
        return events

    def step(self) -> List[Event]:
        """One iteration. Returns the events of this step (also sent to each request's callback)."""
        events: List[Event] = []
        admitted: List[int] = []
        preempted: List[int] = []
        if self._inflight is not None:
            prev, launched, t_launch = self._inflight
            t_plan = time.perf_counter()
            nxt = self._plan_ahead(prev)
            nxt_launched = None
            t_next = time.perf_counter()
            self.stats.plan_ms += (t_next - t_plan) * 1e3
            if nxt is not None:
                try:
                    nxt_launched = self.ex.launch(nxt, after=launched)
                except EngineError:
                    nxt = None
            try:
                sampled = self.ex.collect(launched)
            except EngineError as e:
                for b in prev:
                    self._fail(b.seq, f"forward failed: {e}", events)
                sampled = None
                if nxt_launched is not None:
                    # the batch issued ahead took its tokens from the failed one: wait for it and drop what it made
                    try:
                        self.ex.collect(nxt_launched)
                    except EngineError:
                        pass
                    for b in nxt:
                        if not b.seq.terminal:
                            self._fail(b.seq, f"forward failed: {e}", events)
                    nxt = None
            # a batch's time: from its launch, or from the moment the batch before it was done, to its collection
            now = time.perf_counter()
            self._account(prev, (now - max(t_launch, self._last_done)) * 1e3)
            self._last_done = now
            if sampled is not None:
                self._finish_batch(prev, sampled, events)
            self._inflight = (nxt, nxt_launched, t_next) if nxt is not None else None
            self._retire_finished_now()
            if self._inflight is not None or sampled is None:
                return self._dispatch(events)
            # nothing was issued ahead: go on with an ordinary iteration in this same call
        self._drain_incoming(events)
        self._expire_deadlines(events)
        self._retire(events)
        self._admit(admitted)
        if self.running:
            t_plan = time.perf_counter()
            batch = self._plan(events, preempted)
            self.stats.plan_ms += (time.perf_counter() - t_plan) * 1e3
            if batch and self.lookahead and self.ex.can_launch(batch):
                try:
                    t_launch = time.perf_counter()
                    self._inflight = (batch, self.ex.launch(batch), t_launch)
                except EngineError as e:
                    for b in batch:
                        self._fail(b.seq, f"forward failed: {e}", events)
            elif batch:
                self._run(batch, events)
            step_no = self.stats.steps
            if self.trace is not None:
                self.trace.append(StepTrace(
                    step_no, self._last_rows[0] if batch else 0, self._last_rows[1] if batch else 0,
                    [(b.seq.id, b.start, len(b.tokens), b.sample) for b in batch], preempted, admitted,
                    self.ex.cache.free_pages))
        self._retire_finished_now()
        return self._dispatch(events)

    def _retire_finished_now(self) -> None:
        # Finished requests give their pages back at once rather than at the top of the next
        # step, so that a caller that stops stepping leaves nothing held.
        keep = []
        for seq in self.running:
            if seq.terminal:
                self.ex.end(seq.id)
                self.by_id.pop(seq.id, None)
            else:
                keep.append(seq)
        self.running = keep

    def _account(self, batch: List[BatchItem], ms: float) -> None:
        self.stats.steps += 1
        self._last_forward_ms = ms
        n_decode = sum(1 for b in batch if len(b.tokens) == 1 and b.seq.status == DECODE)
        n_prefill = sum(len(b.tokens) for b in batch) - n_decode
        if n_prefill == 0:
            self.stats.steps_decode_only += 1
            self.stats.forward_decode_only_ms += ms
            self._decode_step_ema_ms = ms if self._decode_step_ema_ms == 0 else 0.8 * self._decode_step_ema_ms + 0.2 * ms
        elif n_decode == 0:
            self.stats.steps_prefill_only += 1
            self.stats.forward_prefill_only_ms += ms
        else:
            self.stats.steps_mixed += 1
            self.stats.forward_mixed_ms += ms
            if self.cfg.decode_protect and self._decode_step_ema_ms > 0:
                # steer the next mixed step's share of prompt rows toward the target multiple of a decode-only step
                target = self.cfg.decode_latency_target * self._decode_step_ema_ms
                if ms > target:
                    self._mixed_prefill_budget = max(min(self.cfg.protected_prefill_min, self.cfg.prefill_token_budget),
                                                     self._mixed_prefill_budget // 2)
                elif ms < 0.5 * target:
                    self._mixed_prefill_budget = min(self.cfg.prefill_token_budget, self._mixed_prefill_budget * 2)
                self.stats.mixed_prefill_budget = self._mixed_prefill_budget
        self.stats.tokens_decoded += n_decode
        self.stats.tokens_prefilled += n_prefill

    def _finish_batch(self, batch: List[BatchItem], sampled: Dict[Hashable, int], events: List[Event]) -> None:
        step_no = self.stats.steps
        for b in batch:
            seq = b.seq
            if seq.terminal:
                continue            # ended (stop token, failure) while this batch was already on its way
            if seq.trace is not None:
                if seq.trace.first_scheduled_s == 0.0:
                    seq.trace.first_scheduled_s = self.clock()
                if b.start < seq.prompt_len:
                    seq.trace.prefill_steps += 1
                    seq.trace.prefill_forward_ms += self._last_forward_ms
            seq.mark_computed(len(b.tokens))
            seq.last_step = step_no
            self.ex.cache.advance(seq.id, seq.num_computed)
            if not b.sample:
                continue
            tok = sampled[seq.id]
            if tok < 0:
                # the executor could not choose a token for this request (its logits are not finite, say); the others
                # of the batch have theirs
                self._fail(seq, "no token could be sampled from the logits (not finite, or of absurd range)", events)
                continue
            if seq.trace is not None and seq.trace.first_token_s == 0.0:
                seq.trace.first_token_s = self.clock()
            seq.append_token(tok)
            if seq.terminal:
                self.stats.finished += 1
                events.append(self._final_event(seq, tok))
            else:
                events.append(Event(seq.id, tok, False, seq.status, None, None, seq.prompt_len, seq.generated))

    def _run(self, batch: List[BatchItem], events: List[Event]) -> None:
        t0 = time.perf_counter()
        try:
            sampled = self.ex.run(batch)
        except EngineError as e:
            # a failed forward fails only this batch's requests (scheduler.cpp:663-666)
            self.stats.steps += 1
            for b in batch:
                self._fail(b.seq, f"forward failed: {e}", events)
            return
        # an executor may say how long its step took (a simulated one in tests); else the wall clock does
        ms = getattr(self.ex, "last_step_ms", None)
        self._account(batch, (time.perf_counter() - t0) * 1e3 if ms is None else ms)
        self._finish_batch(batch, sampled, events)
