"""Generation through the entry point against the plain implementation: greedy, batched == alone,
few pages == many pages, seeded temperature sampling, the command line."""

import os
import subprocess

import numpy as np
import pytest

from plain_llama import PlainLlama, Xoshiro256, sample_temperature
from replay_util import ROOT, random_requests
from tiny_configs import TINY

pytestmark = pytest.mark.gpu


def _engine(folder, dtype="float32", **kw):
    from dynalm_b200 import Engine
    kw.setdefault("ctx", 1024)
    kw.setdefault("batch", 128)
    kw.setdefault("max_running", 8)
    return Engine(folder, dtype=dtype, **kw)


def _check_greedy_against_plain(plain, prompt, generated, slack):
    """Teacher-forced: every generated token has (within `slack`) the largest plain logit."""
    seq = list(prompt) + list(generated)
    logits = plain.logits(seq[:-1])
    for i, tok in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        assert row[tok] >= row.max() - slack, f"token {i}: chose {tok} at {row[tok]:.5f}, best {row.max():.5f}"


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation(name, dtype, slack, tiny_folders):
    cfg = TINY[name][0]
    reqs = random_requests(cfg["vocab_size"], [5, 17, 33], seed=1)
    plain = PlainLlama(tiny_folders[name])
    eng = _engine(tiny_folders[name], dtype)
    outs = eng.generate(list(reqs.values()), max_tokens=16)
    for prompt, g in zip(reqs.values(), outs):
        assert g.status == "finished" and g.finish_reason == "length" and len(g.tokens) == 16
        scale = np.abs(plain.logits(prompt)[-1]).max()
        _check_greedy_against_plain(plain, prompt, g.tokens, slack * max(1.0, scale))
    if dtype == "float32":
        # in 32-bit the plain greedy continuation itself, token by token, up to the first place where the plain
        # implementation's two largest logits are within rounding of each other
        for prompt, g in zip(reqs.values(), outs):
            seq = list(prompt)
            for i, tok in enumerate(g.tokens[:8]):
                row = plain.logits(seq)[-1]
                top = np.sort(row)[-2:]
                if top[1] - top[0] <= 1e-5:
                    break
                assert tok == int(np.argmax(row)), f"token {i} of the continuation: {tok}, plain {int(np.argmax(row))}"
                seq.append(tok)
    # alone == batched: the logits of a request do not depend on what else is in the batch
    alone = [eng.generate(p, max_tokens=16).tokens for p in reqs.values()]
    if dtype == "float32":
        assert alone == [g.tokens for g in outs]
    assert eng.built.cache.free_pages == eng.built.cache.num_pages


def test_few_pages_same_tokens(tiny_folders):
    """An engine with 320 cache tokens gives the same tokens as one with 4096, and preempts."""
    name = "b"
    cfg = TINY[name][0]
    reqs = list(random_requests(cfg["vocab_size"], [40, 90, 17, 100, 64, 33], seed=2).values())
    from dynalm_b200 import SchedulerConfig

    def run(ctx):
        eng = _engine(tiny_folders[name], "float32", ctx=ctx,
                      scheduler=SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                                max_prefill_chunk=32, max_batch_tokens=128))
        out = eng.generate(reqs, max_tokens=40)
        assert eng.built.cache.free_pages == eng.built.cache.num_pages
        return [g.tokens for g in out], eng.scheduler.stats.preemptions

    roomy, p0 = run(4096)
    tight, p1 = run(320)
    assert p0 == 0 and p1 > 0
    assert tight == roomy


def test_temperature_sampling_is_seeded_and_follows_the_walk(tiny_folders):
    name = "b"
    cfg = TINY[name][0]
    prompt = random_requests(cfg["vocab_size"], [23], seed=3)["r0"]
    eng = _engine(tiny_folders[name], "float32")
    a = eng.generate(prompt, max_tokens=24, temperature=0.8, seed=4).tokens
    b = eng.generate(prompt, max_tokens=24, temperature=0.8, seed=4).tokens
    c = eng.generate(prompt, max_tokens=24, temperature=0.8, seed=5).tokens
    assert a == b and a != c
    # teacher-forced: with the same generator the plain walk over plain logits picks the same ids
    plain = PlainLlama(tiny_folders[name])
    rng = Xoshiro256(4)
    logits = plain.logits((prompt + a)[:-1])
    same = sum(sample_temperature(logits[len(prompt) - 1 + i], 0.8, rng.uniform()) == t for i, t in enumerate(a))
    assert same >= len(a) - 1
    # greedy beside sampling in one batch, with filters and penalties
    from dynalm_b200 import SamplingParams
    mixed = eng.generate([prompt, prompt, prompt], max_tokens=12,
                         sampling=[SamplingParams(), SamplingParams(temperature=0.8, seed=4),
                                   SamplingParams(temperature=0.9, top_k=5, top_p=0.9, repetition_penalty=1.1, seed=1)])
    assert mixed[0].tokens == eng.generate(prompt, max_tokens=12).tokens
    assert mixed[1].tokens == a[:12]
    assert len(mixed[2].tokens) == 12


def test_filters_and_penalties_follow_the_reference_pipeline(tiny_folders):
    """Top-k, top-p, min-p and the penalties through the entry point (kernels on the device) against the host's
    pipeline run teacher-forced over the plain implementation's logits with the same generator: the same ids, but
    for a draw that lands within rounding of a boundary."""
    from dynalm_b200 import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    name = "b"
    cfg = TINY[name][0]
    prompt = random_requests(cfg["vocab_size"], [29], seed=5)["r0"]
    eng = _engine(tiny_folders[name], "float32")
    plain = PlainLlama(tiny_folders[name])
    cases = [dict(temperature=0.9, top_k=5), dict(temperature=1.2, top_p=0.9), dict(temperature=0.8, min_p=0.1),
             dict(temperature=1.0, top_k=8, top_p=0.8, repetition_penalty=1.2, frequency_penalty=0.1),
             dict(temperature=0.0, repetition_penalty=1.5, presence_penalty=0.5),
             dict(temperature=0.8, presence_penalty=0.5, penalty_last_n=-1),
             dict(temperature=1.1, top_k=cfg["vocab_size"] + 3, min_p=0.05)]
    params = [SamplingParams(seed=10 + i, **c) for i, c in enumerate(cases)]
    before = eng.executor.host_sampled
    outs = eng.generate([prompt] * len(cases), max_tokens=20, sampling=params)
    assert eng.executor.host_sampled == before           # a vocabulary this small always fits the kernel
    for case, p, out in zip(cases, params, outs):
        a = out.tokens
        assert len(a) == 20
        logits = plain.logits((prompt + a)[:-1]).astype(np.float32)
        host = Sampler(p)
        same = 0
        for i, tok in enumerate(a):
            row = logits[len(prompt) - 1 + i].copy()
            same += host.sample_host(row, prompt + a[:i]) == tok
        assert same >= len(a) - 1, f"{case}: {same} of {len(a)} ids as the host pipeline"
    # and the same request twice gives the same ids
    again = eng.generate([prompt] * len(cases), max_tokens=20, sampling=params)
    assert [o.tokens for o in again] == [o.tokens for o in outs]


def test_a_top_k_beyond_the_kernel_is_finished_on_the_host(tmp_path):
    """Top-k above the 1,024 candidates the filtered kernel keeps: the kernel hands the row back and the host runs the
    pipeline on its logits with the uniform number the kernel was given; beside it in the batch, a request the
    kernel does answer. Both follow the host pipeline over the plain implementation's logits."""
    import torch
    from dynalm_b200 import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    from dynalm_b200.weights import write_model_folder
    cfg = dict(TINY["a"][0], vocab_size=3001)
    write_model_folder(str(tmp_path), cfg, 11, dtype=torch.float32)
    prompt = random_requests(cfg["vocab_size"], [19], seed=6)["r0"]
    eng = _engine(str(tmp_path), "float32")
    plain = PlainLlama(str(tmp_path))
    params = [SamplingParams(temperature=1.0, top_k=2000, top_p=0.95, seed=3), SamplingParams(temperature=1.0, top_k=50, seed=4)]
    assert not Sampler(params[0]).on_device and Sampler(params[1]).on_device
    outs = eng.generate([prompt, prompt], max_tokens=10, sampling=params)
    assert eng.executor.host_sampled == 10
    for p, out in zip(params, outs):
        a = out.tokens
        logits = plain.logits((prompt + a)[:-1]).astype(np.float32)
        host = Sampler(p)
        same = sum(host.sample_host(logits[len(prompt) - 1 + i].copy(), prompt + a[:i]) == tok for i, tok in enumerate(a))
        assert len(a) == 10 and same >= 9, (p, same)


def test_command_line(tiny_folders_bf16):
    proc = subprocess.run([os.path.join(ROOT, "bin", "dynalm"), "run", tiny_folders_bf16["a"], "--tokens", "5,17,3,99",
                           "-n", "8", "--ctx", "256", "--batch", "64", "--no-stream"], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(t) for t in proc.stdout.split()]
    assert len(ids) == 8 and all(0 <= t < 256 for t in ids)
    assert "[stats] prompt 4 tok" in proc.stderr and "finish length" in proc.stderr
    from dynalm_b200 import Engine
    assert Engine(tiny_folders_bf16["a"], ctx=256, batch=64).generate([5, 17, 3, 99], max_tokens=8).tokens == ids


def test_step_function_refusals(tiny_folders):
    from dynalm_b200 import StepEntry
    from dynalm_b200.errors import InvalidArgument, ResourceExhausted
    eng = _engine(tiny_folders["a"], "float32", ctx=64, batch=32, max_running=2)
    with pytest.raises(InvalidArgument, match="no tokens"):
        eng.step([StepEntry("x", [], [])])
    with pytest.raises(InvalidArgument, match="outside"):
        eng.step([StepEntry("x", [1, 256], [0])])
    with pytest.raises(InvalidArgument, match="wants place"):
        eng.step([StepEntry("x", [1, 2], [2])])
    with pytest.raises(InvalidArgument, match="made for 32"):
        eng.step([StepEntry("x", list(range(40)), [0])])
    with pytest.raises(InvalidArgument, match="twice"):
        eng.step([StepEntry("x", [1], [0]), StepEntry("x", [2], [0])])
    eng.step([StepEntry("x", list(range(30)), [29])])
    eng.step([StepEntry("x", list(range(30)), [29])])
    with pytest.raises(ResourceExhausted):
        eng.step([StepEntry("x", list(range(10)), [0])])         # 70 tokens, the pool holds 64
    eng.end("x")
    assert eng.built.cache.free_pages == eng.built.cache.num_pages


@pytest.mark.parametrize("seed", [0, 1])
def test_scheduler_under_random_load_gives_the_tokens_of_each_request_alone(seed, tiny_folders):
    """Forty requests of random lengths, priorities and sampling (greedy or seeded temperature) arrive in bursts
    between steps into an engine with few pages and six running slots; some are cancelled. In 32-bit a row's
    arithmetic does not depend on the batch, so every request that ran to its end must have exactly the tokens it
    gets alone in a roomy engine, whatever was preempted, recomputed or decoded one step ahead around it."""
    from dynalm_b200 import Request, SamplingParams, SchedulerConfig
    name = "b"
    cfg = TINY[name][0]
    rng = np.random.RandomState(40 + seed)
    n = 40
    prompts = [[int(t) for t in rng.randint(0, cfg["vocab_size"], rng.randint(1, 120))] for _ in range(n)]
    new = [int(rng.randint(1, 60)) for _ in range(n)]
    samp = [SamplingParams(temperature=0.8, seed=int(rng.randint(1, 1 << 30))) if rng.rand() < 0.4 else SamplingParams()
            for _ in range(n)]
    prio = [int(rng.randint(0, 3)) for _ in range(n)]

    eng = _engine(tiny_folders[name], "float32", ctx=448, batch=96,
                  scheduler=SchedulerConfig(max_running=6, decode_token_budget=6, prefill_token_budget=64,
                                            max_prefill_chunk=48, max_batch_tokens=96))
    got, ids, cancelled = {}, {}, set()
    submitted = 0
    steps = 0
    while submitted < n or not eng.scheduler.idle:
        if submitted < n and rng.rand() < 0.35:
            for _ in range(int(rng.randint(1, 5))):
                if submitted < n:
                    i = submitted
                    ids[eng.scheduler.submit(Request(prompts[i], new[i], samp[i], priority=prio[i]))] = i
                    got[i] = []
                    submitted += 1
        if rng.rand() < 0.03 and ids:
            rid = int(rng.choice(list(ids)))
            eng.scheduler.cancel(rid)
            cancelled.add(ids[rid])
        for ev in eng.scheduler.step():
            if ev.token is not None:
                got[ids[ev.request_id]].append(ev.token)
            if ev.finished and ev.status == "finished":
                assert ev.completion_tokens == len(got[ids[ev.request_id]])
        steps += 1
        assert steps < 20000
    assert eng.built.cache.free_pages == eng.built.cache.num_pages
    assert eng.scheduler.stats.preemptions > 0, "the pool was meant to be too small"

    alone = _engine(tiny_folders[name], "float32", ctx=4096, batch=128)
    checked = 0
    for i in range(n):
        if i in cancelled:
            continue
        want = alone.generate(prompts[i], max_tokens=new[i], sampling=[samp[i]]).tokens
        assert got[i] == want, f"request {i} (prompt {len(prompts[i])}, {new[i]} new, temperature {samp[i].temperature})"
        checked += 1
    assert checked >= n // 2


def test_cache_size_is_admitted_before_it_is_allocated(tiny_folders):
    """A --ctx that cannot fit the device is refused with the size that would fit, not by an out-of-memory error in
    the middle of the allocation; without a size the cache is sized from the free memory."""
    import torch
    from dynalm_b200 import Engine
    from dynalm_b200.errors import ResourceExhausted
    free = torch.cuda.mem_get_info()[0]
    per_token = 2 * 2 * 2 * 16 * 4             # config a in float32: 2 layers x (k, v) x 2 KV heads x 16 x 4 bytes
    too_many = free // per_token * 2 // 16 * 16
    with pytest.raises(ResourceExhausted, match=r"not enough GPU memory.*use --ctx \d+ or less"):
        Engine(tiny_folders["a"], dtype="float32", ctx=too_many, batch=64, max_running=4)
    assert torch.cuda.mem_get_info()[0] >= free - (256 << 20)          # nothing large was allocated on the way
    eng = Engine(tiny_folders["a"], dtype="float32", batch=64, max_running=4)
    assert eng.built.cache.num_pages * 16 == 65536                      # plenty of memory: the cap of the automatic size
    assert eng.generate([1, 2, 3], max_tokens=4).status == "finished"


def test_engine_thread_serves_submitters_on_other_threads(tiny_folders):
    """The engine runs on its own thread; two threads submit requests while a third reads the streams. Every
    request gets the tokens it gets alone (32-bit: the logits do not depend on what else is in a batch), a stream's
    `next` times out instead of blocking when nothing has come, a cancelled stream ends as cancelled, and after
    shutdown nothing is held."""
    import threading
    name = "b"
    cfg = TINY[name][0]
    reqs = list(random_requests(cfg["vocab_size"], [5, 17, 33, 9, 40, 12, 26, 3], seed=3).values())
    alone_engine = _engine(tiny_folders[name], "float32")
    alone = [alone_engine.generate(p, max_tokens=12).tokens for p in reqs]
    eng = _engine(tiny_folders[name], "float32")
    eng.start()
    streams, lock = {}, threading.Lock()

    def submitter(k):
        for i in range(k, len(reqs), 2):
            st = eng.submit(reqs[i], max_tokens=12)
            with lock:
                streams[i] = st
    got = {}

    def reader():
        while len(got) < len(reqs):
            with lock:
                todo = [(i, st) for i, st in streams.items() if i not in got]
            for i, st in todo:
                got[i] = st.tokens()
    threads = [threading.Thread(target=submitter, args=(k,)) for k in range(2)] + [threading.Thread(target=reader)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
        assert not t.is_alive()
    assert [got[i] for i in range(len(reqs))] == alone
    # nothing submitted: `next` gives up after its timeout; a long request is cancelled in the middle
    long = eng.submit(reqs[2], max_tokens=200)
    first = long.next(timeout=30.0)
    assert first is not None and first.token is not None
    long.cancel()
    rest = list(long)
    assert rest and rest[-1].finished and rest[-1].status == "cancelled" and long.next(timeout=0.01) is None
    # generate() and stream() go through the thread while it runs
    assert eng.generate(reqs[0], max_tokens=12).tokens == alone[0]
    assert [ev.token for ev in eng.stream(reqs[1], max_tokens=12) if ev.token is not None] == alone[1]
    eng.shutdown()
    assert eng.loop_error is None and eng.scheduler.idle
    assert eng.built.cache.free_pages == eng.built.cache.num_pages
