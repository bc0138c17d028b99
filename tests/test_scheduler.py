"""The scheduler's decisions on the CPU, with a fake executor that computes nothing: tokens are a
fixed function of (request's tokens so far), so that recomputation after a preemption must give the
same tokens."""

import hashlib

import torch

from dynalm_b200.errors import EngineError
from dynalm_b200.cache import CacheManager
from dynalm_b200.engine.scheduler import (CANCELLED, ERROR, FINISHED, Request, Scheduler, SchedulerConfig)
from dynalm_b200.parts.base import CacheSpec
from dynalm_b200.sampling import SamplingParams

SPEC = CacheSpec("pages", entry_shape=(1, 16))


class FakeExecutor:
    vocab = 1000

    def __init__(self, kv_tokens=4096, max_requests=8, max_tokens=512, page=16, context=4096):
        self.cache = CacheManager([SPEC], page, kv_tokens, max_requests, context, device=None, dtype=torch.float32)
        self.max_tokens = max_tokens
        self.batches = []
        self.live = set()

    def begin(self, rid):
        self.cache.add_request(rid)
        self.live.add(rid)

    def end(self, rid):
        self.cache.free_request(rid)
        self.live.remove(rid)

    def run(self, batch):
        assert sum(len(b.tokens) for b in batch) <= self.max_tokens
        self.batches.append([(b.seq.id, b.start, len(b.tokens), b.sample) for b in batch])
        out = {}
        for b in batch:
            # the pages for these tokens are there
            assert self.cache.tokens[b.seq.id] >= b.start + len(b.tokens)
            assert b.tokens == b.seq.tokens[b.start:b.start + len(b.tokens)]
            if b.sample:
                h = hashlib.sha256(repr(b.seq.tokens[:b.start + len(b.tokens)]).encode()).digest()
                out[b.seq.id] = int.from_bytes(h[:4], "little") % self.vocab
        self.cache.check()
        return out


class UndecidedExecutor(FakeExecutor):
    """Gives no token (-1) to one request at its third sampled token, as the filtered sampling kernel does for a row
    it cannot sample from."""

    def __init__(self, victim, **kw):
        super().__init__(**kw)
        self.victim, self.seen = victim, 0

    def run(self, batch):
        out = super().run(batch)
        if self.victim in out:
            self.seen += 1
            if self.seen == 3:
                out[self.victim] = -1
        return out


def run_all(s, limit=10000):
    events = []
    n = 0
    while not s.idle:
        events += s.step()
        n += 1
        assert n < limit, "the scheduler does not finish"
    return events


def collect(events):
    toks, final = {}, {}
    for e in events:
        if e.token is not None:
            toks.setdefault(e.request_id, []).append(e.token)
        if e.finished:
            final[e.request_id] = e
    return toks, final


def prompts(n, lens):
    return [[(7 * i + 3 * j) % 1000 for j in range(lens[i % len(lens)])] for i in range(n)]


def test_budgets_order_and_no_skipped_position():
    ex = FakeExecutor()
    cfg = SchedulerConfig(max_running=8, decode_token_budget=4, prefill_token_budget=48, max_prefill_chunk=32,
                          max_batch_tokens=64)
    s = Scheduler(ex, cfg, keep_trace=True)
    ids = [s.submit(Request(p, max_new_tokens=12)) for p in prompts(6, [5, 70, 33, 130, 1, 64])]
    toks, final = collect(run_all(s))
    assert all(final[i].status == FINISHED and final[i].finish_reason == "length" and len(toks[i]) == 12 for i in ids)
    computed = {}
    for batch in ex.batches:
        decode = [b for b in batch if b[2] == 1 and b[3] and computed.get(b[0], 0) > 0]
        assert sum(b[2] for b in batch) <= cfg.max_batch_tokens
        for rid, start, n, sample in batch:
            assert start == computed.get(rid, 0), "a position was skipped or repeated"
            computed[rid] = start + n
    for t in s.trace:
        assert t.decode_rows <= cfg.decode_token_budget and t.prefill_rows <= cfg.prefill_token_budget
        for rid, start, n, sample in t.items:
            if not (n == 1 and sample):
                assert n <= cfg.max_prefill_chunk
    # decode rows come first in a batch
    for batch in ex.batches:
        kinds = [0 if (n == 1 and sample and start > 0) else 1 for _, start, n, sample in batch]
        assert kinds == sorted(kinds)
    assert ex.cache.free_pages == ex.cache.num_pages and not ex.live


def test_decode_rows_rotate_under_a_small_budget():
    ex = FakeExecutor()
    s = Scheduler(ex, SchedulerConfig(max_running=8, decode_token_budget=2, prefill_token_budget=64,
                                      max_prefill_chunk=64, max_batch_tokens=128))
    ids = [s.submit(Request(p, max_new_tokens=6)) for p in prompts(5, [4])]
    toks, final = collect(run_all(s))
    assert all(len(toks[i]) == 6 for i in ids)
    # with 5 decoding and a budget of 2, nobody waits more than 3 steps between tokens
    last = {}
    for n, batch in enumerate(ex.batches):
        for rid, start, k, sample in batch:
            if sample:
                assert n - last.get(rid, n) <= 3
                last[rid] = n


def test_page_shortage_preempts_and_gives_the_same_tokens():
    """An engine with few pages gives the same tokens as a roomy one, and preempts on the way
    (the reference's own check, dynalm/tests/test_engine.cpp:1725-1758)."""
    ps = prompts(6, [40, 90, 17, 120, 64, 33])

    def run(kv):
        ex = FakeExecutor(kv_tokens=kv)
        s = Scheduler(ex, SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                          max_prefill_chunk=32, max_batch_tokens=128), keep_trace=True)
        ids = [s.submit(Request(p, max_new_tokens=40)) for p in ps]
        toks, final = collect(run_all(s))
        assert ex.cache.free_pages == ex.cache.num_pages and not ex.live
        return [toks[i] for i in ids], [final[i].status for i in ids], s

    roomy, st1, s1 = run(4096)
    tight, st2, s2 = run(320)
    assert st1 == st2 == [FINISHED] * 6
    assert s1.stats.preemptions == 0 and s2.stats.preemptions > 0
    assert tight == roomy
    # a preempted request goes to the front of the queue and starts again from position 0
    assert any(t.preempted for t in s2.trace)


def test_a_request_that_can_never_fit_fails_and_others_go_on():
    ex = FakeExecutor(kv_tokens=128, context=4096)
    s = Scheduler(ex, SchedulerConfig(max_running=4, max_batch_tokens=256))
    big = s.submit(Request(list(range(200)), max_new_tokens=4))
    ok = s.submit(Request(list(range(20)), max_new_tokens=4))
    toks, final = collect(run_all(s))
    assert final[big].status == ERROR and "never fit" in final[big].error
    assert final[ok].status == FINISHED and len(toks[ok]) == 4


def test_alone_in_the_pool_and_still_too_big_fails_with_the_reference_message():
    # fits on paper (prompt + new tokens <= pool) but a second request holds pages it cannot take back
    ex = FakeExecutor(kv_tokens=64)
    s = Scheduler(ex, SchedulerConfig(max_running=2, max_batch_tokens=128, prefill_token_budget=64,
                                      max_prefill_chunk=64))
    a = s.submit(Request(list(range(30)), max_new_tokens=30))
    toks, final = collect(run_all(s))
    assert final[a].status == FINISHED        # 60 tokens fit 4 pages


def test_validation_failures():
    ex = FakeExecutor()
    s = Scheduler(ex, SchedulerConfig(context_length=64))
    bad = [s.submit(Request([], 4)), s.submit(Request([1, 2], 0)), s.submit(Request(list(range(60)), 10)),
           s.submit(Request([5, 1000], 4)), s.submit(Request([1], 4, SamplingParams(temperature=-1.0))),
           s.submit(Request([1], 4, SamplingParams(top_p=0.0)))]
    good = s.submit(Request([1, 2, 3], 4))
    toks, final = collect(run_all(s))
    assert all(final[b].status == ERROR for b in bad)
    msgs = [final[b].error for b in bad]
    assert "empty prompt" in msgs[0] and "max_new_tokens" in msgs[1] and "context length" in msgs[2]
    assert "token id" in msgs[3] and "temperature" in msgs[4] and "top_p" in msgs[5]
    assert final[good].status == FINISHED


def test_cancel_stop_token_priority_and_callbacks():
    ex = FakeExecutor()
    s = Scheduler(ex, SchedulerConfig(max_running=1, max_batch_tokens=64))
    seen = []
    low = s.submit(Request([1, 2, 3], 50, priority=0, on_event=seen.append))
    high = s.submit(Request([4, 5, 6], 3, priority=5))
    first = s.step()
    # one slot: the higher priority runs first although it came second
    assert ex.batches[0][0][0] == high
    s.cancel(low)
    toks, final = collect(first + run_all(s))
    assert final[low].status == CANCELLED and final[high].status == FINISHED
    assert seen and seen[-1].finished and seen[-1].status == CANCELLED
    # stop ids end generation with reason eog
    ex2 = FakeExecutor()
    s2 = Scheduler(ex2, SchedulerConfig())
    probe = s2.submit(Request([9, 9, 9], 8))
    t, _ = collect(run_all(s2))
    stop_at = t[probe][2]
    r = s2.submit(Request([9, 9, 9], 8, stop_token_ids=(stop_at,)))
    t2, f2 = collect(run_all(s2))
    assert t2[r] == t[probe][:t[probe].index(stop_at) + 1] and f2[r].finish_reason == "eog"
    assert not ex2.live and ex2.cache.free_pages == ex2.cache.num_pages


def test_admission_waits_for_pages():
    ex = FakeExecutor(kv_tokens=160)          # 10 pages
    s = Scheduler(ex, SchedulerConfig(max_running=4, max_batch_tokens=256, prefill_token_budget=128,
                                      max_prefill_chunk=128), keep_trace=True)
    a = s.submit(Request(list(range(100)), 8))          # 7 pages + headroom
    b = s.submit(Request(list(range(60)), 8))           # needs 4 + 1: must wait for a
    s.step()
    assert [q.id for q in s.running] == [a] and [q.id for q in s.waiting] == [b]
    toks, final = collect(run_all(s))
    assert final[a].status == final[b].status == FINISHED


class FakeAsyncExecutor(FakeExecutor):
    """The fake with `launch` / `collect`, as the GPU executor has them: a decode batch is issued without its
    tokens being known, and the batch after it may be issued before the first is collected."""

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.launched = 0
        self.ahead = 0

    @staticmethod
    def can_launch(batch):
        return bool(batch) and all(b.sample and len(b.tokens) == 1 for b in batch)

    def launch(self, batch, after=None):
        assert self.can_launch(batch)
        self.launched += 1
        self.ahead += after is not None
        self.batches.append([(b.seq.id, b.start, 1, True) for b in batch])
        for b in batch:
            assert self.cache.tokens[b.seq.id] >= b.start + 1
        return [(b.seq, b.start) for b in batch]

    def collect(self, handle):
        out = {}
        for seq, start in handle:
            assert len(seq.tokens) == start + 1, "the token before this one has not been resolved"
            h = hashlib.sha256(repr(seq.tokens[:start + 1]).encode()).digest()
            out[seq.id] = int.from_bytes(h[:4], "little") % self.vocab
        return out


def test_decoding_one_step_ahead_gives_the_same_tokens():
    ps = prompts(5, [12, 40, 7, 33, 20])

    def run(ex, stop=()):
        s = Scheduler(ex, SchedulerConfig(max_running=8, decode_token_budget=8, prefill_token_budget=64,
                                          max_prefill_chunk=32, max_batch_tokens=128))
        ids = [s.submit(Request(p, max_new_tokens=10 + 3 * i, stop_token_ids=stop)) for i, p in enumerate(ps)]
        toks, final = collect(run_all(s))
        assert not ex.live and ex.cache.free_pages == ex.cache.num_pages
        return [toks[i] for i in ids], [final[i].finish_reason for i in ids]

    plain_toks, plain_reasons = run(FakeExecutor())
    ex = FakeAsyncExecutor()
    ahead_toks, ahead_reasons = run(ex)
    assert ahead_toks == plain_toks and ahead_reasons == plain_reasons == ["length"] * 5
    assert ex.ahead > 10                                  # most decode batches were issued before the previous one was collected
    # no request is ever issued past its last token
    per_req = {}
    for batch in ex.batches:
        for rid, start, n, _ in batch:
            per_req[rid] = max(per_req.get(rid, 0), start + n)
    for i, p in enumerate(ps):
        assert per_req[i + 1] == len(p) + 10 + 3 * i - 1
    # a stop token ends a request although the batch after it is already on its way; the others go on unharmed
    stop = (plain_toks[1][4],)
    want_toks, want_reasons = run(FakeExecutor(), stop)
    got_toks, got_reasons = run(FakeAsyncExecutor(), stop)
    assert got_toks == want_toks and got_reasons == want_reasons and "eog" in got_reasons


def test_a_failed_step_with_a_batch_in_flight_fails_both_and_frees_everything():
    """The GPU executor finds a step's status word in the copy of its chosen ids and raises when a kernel gave up a
    wait. By then the next batch has been issued from the failed one's tokens: its requests fail too, nothing of it
    is emitted, every page comes back, and requests submitted afterwards run normally."""
    class Failing(FakeAsyncExecutor):
        fail_at = 6

        def collect(self, handle):
            self.collected = getattr(self, "collected", 0) + 1
            if self.collected == self.fail_at:
                raise EngineError("a kernel gave up waiting on a barrier (status 3); the step's results are not valid")
            if self.collected == self.fail_at + 1:
                return {}            # the batch that was in flight behind the failed one: waited for, nothing kept
            return super().collect(handle)

    ex = Failing()
    s = Scheduler(ex, SchedulerConfig(max_running=8, decode_token_budget=8, prefill_token_budget=64,
                                      max_prefill_chunk=32, max_batch_tokens=128))
    ids = [s.submit(Request(p, max_new_tokens=20)) for p in prompts(3, [12, 20, 7])]
    toks, final = collect(run_all(s))
    assert all(final[i].status == "error" and "gave up waiting" in final[i].error for i in ids)
    assert all(len(toks[i]) < 20 for i in ids)
    assert not ex.live and ex.cache.free_pages == ex.cache.num_pages and s.idle
    ex.cache.check()
    again = s.submit(Request(prompts(1, [9])[0], max_new_tokens=5))
    toks, final = collect(run_all(s))
    assert final[again].status == FINISHED and len(toks[again]) == 5


def test_a_request_without_a_token_fails_alone_with_a_batch_in_flight():
    """One step ahead: the batch after the one in which a request got no token (-1) is on its way already, with a
    row of that request in it; the request fails, that row's result is dropped, and the others get the tokens they
    get without it."""
    class Undecided(FakeAsyncExecutor):
        victim, seen = None, 0

        def collect(self, handle):
            handle = [(seq, start) for seq, start in handle if not seq.terminal]
            out = super().collect(handle)
            if self.victim in out:
                self.seen += 1
                if self.seen == 4:
                    out[self.victim] = -1
            return out

    ps = prompts(3, [12, 20, 7])

    def run(ex, which=None):
        s = Scheduler(ex, SchedulerConfig(max_running=8, decode_token_budget=8, prefill_token_budget=64,
                                          max_prefill_chunk=32, max_batch_tokens=128))
        ids = [s.submit(Request(p, max_new_tokens=12)) for p in ps]
        if which is not None:
            ex.victim = ids[which]
        toks, final = collect(run_all(s))
        assert not ex.live and ex.cache.free_pages == ex.cache.num_pages
        return [toks[i] for i in ids], [final[i] for i in ids]

    want, _ = run(FakeAsyncExecutor())
    ex = Undecided()
    got, final = run(ex, which=1)
    assert ex.ahead > 5
    assert final[1].status == "error" and "no token could be sampled" in final[1].error
    assert got[1] == want[1][:len(got[1])] and len(got[1]) < 12
    assert got[0] == want[0] and got[2] == want[2] and final[0].status == final[2].status == FINISHED


def test_one_step_ahead_with_arrivals_cancels_and_few_pages():
    """Requests arriving, being cancelled and being preempted while batches are in flight: the scheduler falls
    back to the ordinary iteration whenever the steady state does not hold, and the tokens stay the same."""
    ps = prompts(6, [40, 90, 17, 120, 64, 33])

    def run(ex):
        s = Scheduler(ex, SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                          max_prefill_chunk=32, max_batch_tokens=128))
        ids = [s.submit(Request(p, max_new_tokens=40)) for p in ps[:3]]
        events = []
        for n in range(10000):
            if s.idle:
                break
            events += s.step()
            if n == 6:
                ids += [s.submit(Request(p, max_new_tokens=40)) for p in ps[3:]]
            if n == 30:
                s.cancel(ids[2])
        toks, final = collect(events)
        assert not ex.live and ex.cache.free_pages == ex.cache.num_pages
        return [toks.get(i, []) for i in ids], [final[i].status for i in ids], s.stats.preemptions

    roomy = run(FakeExecutor(kv_tokens=4096))
    ahead_roomy = run(FakeAsyncExecutor(kv_tokens=4096))
    ahead_tight = run(FakeAsyncExecutor(kv_tokens=320))
    for got in (ahead_roomy, ahead_tight):
        for i in (0, 1, 3, 4, 5):
            assert got[0][i] == roomy[0][i] and got[1][i] == FINISHED
        assert got[1][2] == CANCELLED and got[0][2] == roomy[0][2][:len(got[0][2])]
    assert ahead_tight[2] > 0


def test_deadlines_fail_running_and_queued_requests():
    """A request past its timeout fails with the reference's messages, whether it is running or still queued
    (dynalm/src/scheduler/scheduler.cpp:293-309); its pages come back; the others go on."""
    now = [0.0]
    ex = FakeExecutor(kv_tokens=64, max_requests=4)                      # room for one 40-token request at a time
    s = Scheduler(ex, SchedulerConfig(max_running=4, prefill_token_budget=16, max_prefill_chunk=16, max_batch_tokens=64),
                  clock=lambda: now[0])
    a = s.submit(Request(list(range(40)), max_new_tokens=8, timeout_ms=50))
    b = s.submit(Request(list(range(40)), max_new_tokens=8, timeout_ms=20))   # waits behind a: no pages for both
    c = s.submit(Request(list(range(40)), max_new_tokens=2))
    events = s.step()
    assert [q.id for q in s.running] == [a] and len(s.waiting) == 2
    now[0] = 0.030                                                        # b's deadline passes in the queue
    events = s.step()
    failed = [e for e in events if e.finished]
    assert [(e.request_id, e.status, e.error) for e in failed] == [(b, "error", "request timed out while queued")]
    now[0] = 0.060                                                        # a's passes while it runs
    events = s.step()
    failed = [e for e in events if e.finished]
    assert [(e.request_id, e.status, e.error) for e in failed] == [(a, "error", "request timed out")]
    assert a not in ex.live
    events = run_all(s)
    done = [e for e in events if e.finished]
    assert [(e.request_id, e.status, e.completion_tokens) for e in done] == [(c, "finished", 2)]
    assert s.stats.timed_out == 2 and ex.cache.free_pages == ex.cache.num_pages


def test_decode_protected_prefill_budget_halves_and_doubles():
    """Beside decode rows the prompt rows follow the adaptive budget: it halves after a mixed step that took more than
    decode_latency_target x a decode-only step, down to protected_prefill_min, and doubles again after fast ones;
    steps without decode rows keep the whole budget (dynalm/src/scheduler/scheduler.h:138-150)."""
    ex = FakeExecutor(kv_tokens=8192, max_requests=8, max_tokens=512, context=8192)
    ms_per_prompt_row = [1.0]

    real_run = ex.run

    def run(batch):
        rows = sum(len(b.tokens) for b in batch if len(b.tokens) > 1)
        ex.last_step_ms = 1.0 + ms_per_prompt_row[0] * rows            # a decode-only step costs 1 ms
        return real_run(batch)
    ex.run = run
    cfg = SchedulerConfig(max_running=8, decode_token_budget=8, prefill_token_budget=256, max_prefill_chunk=0,
                          max_batch_tokens=512, protected_prefill_min=32, decode_latency_target=6.0)
    s = Scheduler(ex, cfg)
    s.submit(Request(list(range(10)), max_new_tokens=400))
    for _ in range(4):
        s.step()                                                         # prompt, then decode-only steps: 1 ms each
    assert s.stats.steps_decode_only >= 2
    s.submit(Request([t % 1000 for t in range(3000)], max_new_tokens=4))
    budgets, prompt_rows = [], []
    for _ in range(6):
        s.step()
        prompt_rows.append(sum(n for _, _, n, _ in ex.batches[-1] if n > 1))
        budgets.append(s.stats.mixed_prefill_budget)
    # 256 prompt rows cost 257 ms > 6 ms: the budget halves step after step down to its floor
    assert prompt_rows[:5] == [256, 128, 64, 32, 32] and budgets[:4] == [128, 64, 32, 32]
    ms_per_prompt_row[0] = 0.01                                          # prompt rows become cheap: 1.32 ms < 3 ms
    for _ in range(4):
        s.step()
        budgets.append(s.stats.mixed_prefill_budget)
    assert budgets[-4:] == [64, 128, 256, 256]
    cfg.decode_protect = False
    s.step()
    assert sum(n for _, _, n, _ in ex.batches[-1] if n > 1) == 256


def test_a_failed_forward_fails_its_batch_only_and_gives_the_pages_back():
    """The executor raises for one step (as a kernel that reports an error does): the requests of that batch end
    with an error that names it, their pages are free again, and requests submitted afterwards run as usual
    (dynalm/src/scheduler/scheduler.cpp:663-666)."""
    from dynalm_b200.errors import EngineError

    class FailsOnce(FakeExecutor):
        fail_at = 3

        def run(self, batch):
            self.fail_at -= 1
            if self.fail_at == 0:
                raise EngineError("a product gave up waiting on a barrier")
            return super().run(batch)

    ex = FailsOnce(kv_tokens=1024)
    s = Scheduler(ex, SchedulerConfig(max_running=4, max_batch_tokens=256))
    first = [s.submit(Request(p, max_new_tokens=6)) for p in prompts(3, [20, 33, 7])]
    events = run_all(s)
    toks, final = collect(events)
    failed = [r for r in first if final[r].status == ERROR]
    assert failed, "the failing step held at least one request"
    for r in failed:
        assert "forward failed" in final[r].error and "barrier" in final[r].error
    for r in first:
        if r not in failed:
            assert final[r].status == FINISHED and len(toks[r]) == 6
    assert not ex.live and ex.cache.free_pages == ex.cache.num_pages
    ex.cache.check()
    later = s.submit(Request(list(range(40)), max_new_tokens=5))
    toks, final = collect(run_all(s))
    assert final[later].status == FINISHED and len(toks[later]) == 5
    # the time split of the reference's SchedulerStats (scheduler.h:260-313): planning and callbacks on the host
    assert s.stats.plan_ms > 0.0 and s.stats.emit_ms == 0.0               # nobody asked for callbacks
    seen = []
    s.submit(Request(list(range(12)), max_new_tokens=3, on_event=seen.append))
    run_all(s)
    assert len(seen) == 3 and seen[-1].finished and s.stats.emit_ms > 0.0


def test_a_lone_prompt_gets_the_solo_chunk():
    """solo_prefill_chunk (dynalm/src/scheduler/scheduler.cpp:436-472): a step without decode rows with exactly one
    request prefilling gives it the larger portion; two prompts prefilling get the regular portions unless the solo
    budget is split; steps with decode rows are as ever. The tokens are the same either way."""
    def rows(ex):
        return [[(n, sample) for _, _, n, sample in b] for b in ex.batches]

    base = dict(max_running=4, max_batch_tokens=512, prefill_token_budget=64, max_prefill_chunk=32)
    ex = FakeExecutor()
    s = Scheduler(ex, SchedulerConfig(solo_prefill_chunk=200, **base))
    a = s.submit(Request(list(range(450)), max_new_tokens=3))
    toks_solo, _ = collect(run_all(s))
    assert [b[0][0] for b in rows(ex)[:3]] == [200, 200, 50]          # 450 = 200 + 200 + 50, then decoding
    assert s.stats.steps_solo_prefill == 3
    ex0 = FakeExecutor()
    s0 = Scheduler(ex0, SchedulerConfig(**base))
    a0 = s0.submit(Request(list(range(450)), max_new_tokens=3))
    toks_plain, _ = collect(run_all(s0))
    assert toks_solo[a] == toks_plain[a0] and rows(ex0)[0] == [(32, False)] and s0.stats.steps_solo_prefill == 0

    # two prompts prefilling: regular portions under the regular budget ...
    ex2 = FakeExecutor()
    s2 = Scheduler(ex2, SchedulerConfig(solo_prefill_chunk=200, **base))
    s2.submit(Request(list(range(100)), max_new_tokens=2))
    s2.submit(Request(list(range(100, 190)), max_new_tokens=2))
    run_all(s2)
    assert rows(ex2)[0] == [(32, False), (32, False)]
    # ... or the solo budget shared among them
    ex3 = FakeExecutor()
    s3 = Scheduler(ex3, SchedulerConfig(solo_prefill_chunk=200, solo_prefill_split=True, **base))
    s3.submit(Request(list(range(150)), max_new_tokens=2))
    s3.submit(Request(list(range(100, 250)), max_new_tokens=2))
    run_all(s3)
    assert rows(ex3)[0] == [(100, False), (100, False)]

    # beside a decoding request a new prompt gets the regular portion
    ex4 = FakeExecutor()
    s4 = Scheduler(ex4, SchedulerConfig(solo_prefill_chunk=200, **base))
    s4.submit(Request(list(range(10)), max_new_tokens=30))
    for _ in range(3):
        s4.step()
    s4.submit(Request(list(range(300)), max_new_tokens=2))
    run_all(s4)
    mixed = [b for b in rows(ex4) if len(b) == 2]
    assert mixed and all(b[1][0] <= 32 for b in mixed if b[0] == (1, True))


def test_request_traces_tell_each_request_s_life():
    """With traces kept, every request leaves a record when it ends (dynalm/src/scheduler/scheduler.h:113-125):
    its times in order, the steps that computed prompt rows (again after a preemption), how it ended."""
    tick = [0.0]

    def clock():
        tick[0] += 0.001
        return tick[0]

    ps = prompts(6, [40, 90, 17, 120, 64, 33])
    ex = FakeExecutor(kv_tokens=320)
    s = Scheduler(ex, SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                      max_prefill_chunk=32, max_batch_tokens=128), keep_trace=True, clock=clock)
    ids = [s.submit(Request(p, max_new_tokens=40)) for p in ps]
    bad = s.submit(Request([5, 6, 7], max_new_tokens=0))                   # refused at validation
    run_all(s)
    traces = {t.id: t for t in s.request_traces}
    assert sorted(traces) == sorted(ids + [bad]) and len(s.request_traces) == 7
    assert traces[bad].status == ERROR and traces[bad].first_token_s == 0.0 and traces[bad].admit_s == 0.0
    assert traces[bad].submit_s < traces[bad].finish_s
    assert s.stats.preemptions > 0 and sum(t.preemptions for t in traces.values()) == s.stats.preemptions
    for rid, p in zip(ids, ps):
        t = traces[rid]
        assert t.status == FINISHED and t.prompt_tokens == len(p) and t.generated == 40
        assert 0.0 < t.submit_s < t.admit_s < t.first_scheduled_s <= t.first_token_s < t.finish_s
        least = -(-len(p) // 32)
        assert t.prefill_steps >= least and (t.preemptions > 0 or t.prefill_steps == least)
        assert t.prefill_forward_ms >= 0.0
    assert any(t.preemptions > 0 and t.prefill_steps > -(-t.prompt_tokens // 32) for t in traces.values())
    # without traces nothing is kept
    s0 = Scheduler(FakeExecutor(), SchedulerConfig())
    s0.submit(Request([1, 2, 3], max_new_tokens=2))
    run_all(s0)
    assert s0.request_traces is None and s0.trace is None


def test_engine_stats_snapshot_names_how_steps_were_issued():
    """Engine.stats() on stand-ins (no GPU): the scheduler's counters, the cache's pages and how the steps were
    issued (launches, library products, layers issued by address, graphs)."""
    from types import SimpleNamespace
    from dynalm_b200.engine.engine import Engine
    from dynalm_b200.engine.scheduler import SchedulerStats
    eng = Engine.__new__(Engine)
    eng.scheduler = SimpleNamespace(stats=SchedulerStats(steps=3))
    eng.built = SimpleNamespace(cache=SimpleNamespace(free_pages=5, num_pages=8, bytes=lambda: 1024),
                                runtime=SimpleNamespace(workspace_bytes=lambda: 2048))
    eng.step_fn = SimpleNamespace(graph_captures=2, graph_capture_ms=9.87654, graph_kernel_launches=232)
    got = eng.stats()
    assert got["scheduler"]["steps"] == 3 and got["free_pages"] == 5 and got["pages"] == 8
    assert got["graphs"] == {"captured": 2, "capture_ms": 9.877, "replayed_kernel_launches": 232}
    assert {"kernel_launches", "library_products", "layers_issued_by_address", "cache_bytes", "workspace_bytes"} <= set(got)


def test_submit_and_cancel_from_other_threads():
    """Four threads submit (and one of them cancels) while this thread steps: every request ends exactly once, the
    ones that were not cancelled with the tokens they get alone, and nothing stays held."""
    import threading
    ps = prompts(24, [10 + 3 * (i % 7) for i in range(24)])
    alone = {}
    for i, p in enumerate(ps):
        s1 = Scheduler(FakeExecutor(), SchedulerConfig(max_running=8, max_batch_tokens=128))
        rid = s1.submit(Request(p, max_new_tokens=6))
        alone[i] = collect(run_all(s1))[0][rid]
    ex = FakeAsyncExecutor()
    s = Scheduler(ex, SchedulerConfig(max_running=8, decode_token_budget=8, prefill_token_budget=64,
                                      max_prefill_chunk=32, max_batch_tokens=128))
    rid_of, cancelled, lock = {}, set(), threading.Lock()

    def worker(k):
        for i in range(k, len(ps), 4):
            rid = s.submit(Request(ps[i], max_new_tokens=6))
            with lock:
                rid_of[i] = rid
            if k == 3 and i % 8 == 3:
                s.cancel(rid)
                with lock:
                    cancelled.add(i)
    threads = [threading.Thread(target=worker, args=(k,)) for k in range(4)]
    for t in threads:
        t.start()
    events = []
    while any(t.is_alive() for t in threads) or not s.idle:
        events += s.step()
    for t in threads:
        t.join()
    toks, final = collect(events)
    assert sorted(final) == sorted(rid_of.values())
    assert sum(1 for e in events if e.finished) == len(ps)
    for i, rid in rid_of.items():
        if i in cancelled:
            assert final[rid].status in (CANCELLED, FINISHED)
        else:
            assert final[rid].status == FINISHED and toks[rid] == alone[i]
    assert not ex.live and ex.cache.free_pages == ex.cache.num_pages
    ex.cache.check()


def test_a_request_without_a_token_fails_alone():
    ex = UndecidedExecutor(victim=None)
    s = Scheduler(ex, SchedulerConfig(max_running=4))
    ids = [s.submit(Request(p, 6)) for p in prompts(3, [5, 9, 4])]
    ex.victim = ids[1]
    toks, final = collect(run_all(s))
    assert final[ids[1]].status == "error" and "no token could be sampled" in final[ids[1]].error
    assert len(toks[ids[1]]) == 2
    assert all(final[i].status == "finished" and len(toks[i]) == 6 for i in (ids[0], ids[2]))
    assert ex.cache.free_pages == ex.cache.num_pages and not ex.live
