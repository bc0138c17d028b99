"""Replay on the GPU against the plain implementation: the same requests whole, with the last 32
tokens one by one, in portions of changing size, and mixed with so few pages that they are reused;
in 32-bit and in bfloat16, for every tiny configuration."""

import numpy as np
import pytest

from plain_llama import PlainLlama
from replay_util import (compare, kl_and_top1, plan_chunks, plan_many_rows, plan_mixed, plan_tail, plan_whole,
                         random_requests, run_plan_in_process, run_plan_trace_run)
from tiny_configs import TINY

pytestmark = pytest.mark.gpu

# (absolute, relative-to-row-scale) tolerance on logits per dtype
# The bfloat16 engine is compared with the plain implementation on the same bfloat16 weights; what is left is the
# rounding of activations: at most 0.0048 over all configurations and plans when this was set, so three times that.
TOL = {"float32": (2e-5, 2e-5), "bfloat16": (1.4e-2, 0.0)}
# The plain and the engine's distributions: mean KL over the written rows at most this, and the same most likely
# token wherever the plain implementation's two largest logits are further apart than NEAR_TIE
# (the reference's gate on its own GPU path is a mean KL of 0.0025, dynalm/benchmarks/bench_gpu_accuracy.cpp:91-92).
# Here the logits are small (a tiny random model) and the largest mean KL seen was 3.6e-7 in bfloat16 and 5e-15 in
# 32-bit, so the gates are three times those.
KL_GATE = {"float32": 1e-12, "bfloat16": 1.2e-6}
NEAR_TIE = {"float32": 1e-5, "bfloat16": 5e-2}
LENGTHS = {"a": [5, 17, 33, 70, 41, 64], "b": [1, 7, 40, 64, 100, 129], "c": [3, 48, 95, 33, 160, 16],
           "d": [2, 65, 130, 31, 16], "e": [4, 150, 33, 260, 71, 129], "f": [2, 140, 66, 17, 200],
           "g": [3, 50, 97, 18, 140, 64]}
SIZES = [16, 7, 2, 5, 3, 2, 11, 32, 2, 9]


@pytest.fixture(scope="module")
def folders(tiny_folders, tiny_folders_bf16):
    """dtype -> name -> model folder whose file holds that dtype: the bfloat16 engine and the plain implementation
    it is compared with read the same bfloat16 weights, so that what is left between them is the rounding of
    activations, not of weights."""
    return {"float32": tiny_folders, "bfloat16": tiny_folders_bf16}


@pytest.fixture(scope="module")
def plain_logits(folders):
    """(name, dtype) -> (requests, plain logits of every request), made when first asked for."""
    made = {}

    class Lookup:
        def __getitem__(self, key):
            name, dtype = key
            if key not in made:
                reqs = random_requests(TINY[name][0]["vocab_size"], LENGTHS[name], seed=11 + len(name))
                model = PlainLlama(folders[dtype][name])
                made[key] = (reqs, {r: model.logits(t) for r, t in reqs.items()})
            return made[key]
    return Lookup()


def _built(folder, dtype, kv_tokens, max_batch):
    from dynalm_b200.engine import build
    return build(folder, dtype=dtype, kv_tokens=kv_tokens, max_batch_tokens=max_batch, max_requests=8,
                 context=max(kv_tokens, 256))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e", "f", "g"])
def test_replay_all_cuts(name, dtype, folders, plain_logits):
    reqs, plain = plain_logits[name, dtype]
    tol = TOL[dtype]
    plans = {
        "whole": plan_whole(reqs),
        "tail32": plan_tail(reqs, 32),
        "chunks": plan_chunks(reqs, SIZES),
        "mixed": plan_mixed(reqs, seed=5),
        "mixed2": plan_mixed(reqs, seed=6, max_live=3, decode_tail=20),
    }
    for what, plan in plans.items():
        # the pool is just what the plan needs, so that finished requests' pages are reused
        need = plan.max_live_tokens(64)
        built = _built(folders[dtype][name], dtype, need, max(need, 64))
        got = run_plan_in_process(built.step_fn, plan)
        worst = compare(plan, got, plain, tol[0], tol[1], f"{name}/{dtype}/{what}")
        assert built.cache.free_pages == built.cache.num_pages, "pages were lost"
        kl, top1 = kl_and_top1(plan, got, plain, near_tie=NEAR_TIE[dtype])
        print(f"{name} {dtype} {what}: steps {len(plan.steps)} pool {need} worst {worst:.3g} KL {kl:.3g} top-1 {top1:.4f}")
        assert kl <= KL_GATE[dtype] and top1 == 1.0, f"{name}/{dtype}/{what}: mean KL {kl:.3g}, top-1 agreement {top1:.4f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "e", "g"])
def test_many_single_token_rows(name, dtype, folders):
    """36 short requests alive at once: steps of 17 to 36 single-token rows, beside a prompt portion and alone. In
    bfloat16 these are the row counts at which the matrix products leave the weight-streaming kernels (the library
    product and the separate activation kernel where the tensor-core product has too few tiles) and at which the
    decode attention merges its key splits through scratch memory instead of inside a thread-block cluster."""
    from dynalm_b200.engine import build
    from dynalm_b200.kernels import gemm
    cfg = TINY[name][0]
    rng = np.random.RandomState(40)
    short = random_requests(cfg["vocab_size"], [int(n) for n in rng.randint(24, 71, size=36)], seed=41)
    long = {"L" + r: t for r, t in random_requests(cfg["vocab_size"], [150, 91], seed=42).items()}
    model = PlainLlama(folders[dtype][name])
    plain = {r: model.logits(t) for r, t in {**short, **long}.items()}
    plan = plan_many_rows(short, long, seed=43)
    rows_per_step = [sum(1 for e in st["entries"] if len(e["tokens"]) == 1) for st in plan.steps]
    assert max(rows_per_step) == 36 and sum(1 for n in rows_per_step if 17 <= n <= 40) >= 10
    need = plan.max_live_tokens(64)
    before = gemm.LIBRARY_CALLS
    built = build(folders[dtype][name], dtype=dtype, kv_tokens=need, max_batch_tokens=320, max_requests=40, context=256)
    got = run_plan_in_process(built.step_fn, plan)
    worst = compare(plan, got, plain, *TOL[dtype], f"many/{name}/{dtype}")
    kl, top1 = kl_and_top1(plan, got, plain, near_tie=NEAR_TIE[dtype])
    print(f"many {name} {dtype}: steps {len(plan.steps)} pool {need} worst {worst:.3g} KL {kl:.3g} top-1 {top1:.4f}")
    assert kl <= KL_GATE[dtype] and top1 == 1.0
    assert built.cache.free_pages == built.cache.num_pages, "pages were lost"
    if dtype == "bfloat16":
        assert gemm.LIBRARY_CALLS > before, "no step took the path of 17 to 127 rows"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, folders, plain_logits, tmp_path):
    """The program itself, as a user runs it: stdin in, files out, `done` lines."""
    name = "b"
    reqs, plain = plain_logits[name, dtype]
    plan = plan_mixed(reqs, seed=7)
    vocab = TINY[name][0]["vocab_size"]
    summary = str(tmp_path / "summary.txt")
    got = run_plan_trace_run(folders[dtype][name], dtype, plan, str(tmp_path / "out"), plan.max_live_tokens(64), vocab,
                             summary=summary)
    compare(plan, got, plain, *TOL[dtype], f"trace_run/{dtype}")
    # the text summary describes the files: one line per wanted place, the largest logit and the row's sums
    lines = open(summary).read().splitlines()
    assert len(lines) == sum(len(rows) for rows in plan.rows.values())
    first_step = min(plan.rows)
    words = lines[0].split()
    assert words[:2] == ["step", str(first_step)] and words[6] == "argmax"
    row = got[first_step][0]
    assert int(words[7]) == int(np.argmax(row))
    assert abs(float(words[-2]) - float(row.astype(np.float64).sum())) <= 1e-3 * max(1.0, abs(float(row.sum())))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders):
    """A short prompt and 380 tokens decoded one by one (pages fill and new ones are taken every 16
    steps; in bfloat16 the decode steps replay a CUDA graph whose key changes as the context grows)."""
    name = "c"
    cfg = TINY[name][0]
    toks = random_requests(cfg["vocab_size"], [400], seed=21)["r0"]
    plain = {"r0": PlainLlama(folders[dtype][name]).logits(toks)}
    plan = plan_tail({"r0": toks}, tail=380)
    built = _built(folders[dtype][name], dtype, 448, 64)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, plain, *TOL[dtype], f"long/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_first_tokens_of_a_sequence(name, dtype, folders):
    """Requests of one, two and three tokens: position 0 alone, and the first steps from it."""
    cfg = TINY[name][0]
    reqs = random_requests(cfg["vocab_size"], [1, 2, 3, 2], seed=22)
    model = PlainLlama(folders[dtype][name])
    plain = {r: model.logits(t) for r, t in reqs.items()}
    for what, plan in (("whole", plan_whole(reqs)), ("one by one", plan_tail(reqs, 32)),
                       ("together", plan_mixed(reqs, seed=1, decode_tail=1, sizes=(2, 3)))):
        built = _built(folders[dtype][name], dtype, 256, 64)
        compare(plan, run_plan_in_process(built.step_fn, plan), plain, *TOL[dtype], f"first/{name}/{dtype}/{what}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "e"])
def test_fork_and_copy_on_write_match_from_scratch(name, dtype, folders):
    """A prompt that ends in the middle of a page is forked twice; the three requests go on with different tokens
    (one by one, in portions of three, and in one piece) in the same steps. Each must give the logits of its own
    whole sequence computed from scratch: the shared half page is copied before the first write into it."""
    from dynalm_b200.engine import StepEntry
    cfg = TINY[name][0]
    rng = np.random.RandomState(31)
    base = [int(t) for t in rng.randint(0, cfg["vocab_size"], 41)]
    tails = {"p": [int(t) for t in rng.randint(0, cfg["vocab_size"], 30)],
             "q": [int(t) for t in rng.randint(0, cfg["vocab_size"], 27)],
             "r": [int(t) for t in rng.randint(0, cfg["vocab_size"], 12)]}
    model = PlainLlama(folders[dtype][name])
    plain = {r: model.logits(base + t) for r, t in tails.items()}
    built = _built(folders[dtype][name], dtype, 256, 64)
    fn = built.step_fn
    tol = TOL[dtype]

    def close(got, want, what):
        err = np.abs(got - want).max()
        assert err <= tol[0] + tol[1] * np.abs(want).max(), f"{what}: {err}"

    got = fn.step([StepEntry("p", base, [40])]).float().cpu().numpy()
    close(got[0], plain["p"][40], "prompt")
    free_before = built.cache.free_pages
    fn.fork("p", "q")
    fn.fork("p", "r")
    assert built.cache.free_pages == free_before            # a fork takes no page
    built.cache.check()
    done = {"p": 0, "q": 0, "r": 0}
    portion = {"p": 1, "q": 3, "r": 12}
    while any(done[r] < len(tails[r]) for r in tails):
        entries, places = [], []
        for r in ("q", "p", "r"):
            n = min(portion[r], len(tails[r]) - done[r])
            if n <= 0:
                continue
            entries.append(StepEntry(r, tails[r][done[r]:done[r] + n], list(range(n))))
            places.append((r, done[r], n))
            done[r] += n
        got = fn.step(entries).float().cpu().numpy()
        row = 0
        for r, start, n in places:
            for i in range(n):
                close(got[row], plain[r][41 + start + i], f"{r} token {start + i}")
                row += 1
        built.cache.check()
    for r in tails:
        fn.end(r)
    built.cache.check()
    assert built.cache.free_pages == built.cache.num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["b", "d", "e", "g"])
def test_layers_issued_by_address_give_the_same_bits(name, dtype, folders, plain_logits, monkeypatch):
    """From the third layer on, a step re-issues the second layer's launches with the layer's own addresses put in
    (engine/launch_memo.py) instead of going through the parts' Python code: the logits are the same bits as with
    every layer run through its parts, in whole prompts, portions and mixed steps; and the short way was taken
    (also where a layer's products go to the library: config d in bfloat16, whose width is no multiple of 8)."""
    from dynalm_b200.engine import launch_memo
    reqs, _ = plain_logits[name, dtype]
    for what, plan in (("chunks", plan_chunks(reqs, SIZES)), ("mixed", plan_mixed(reqs, seed=5))):
        need = plan.max_live_tokens(64)
        got = {}
        for enabled in (True, False):
            monkeypatch.setattr(launch_memo, "ENABLED", enabled)
            before = launch_memo.REPLAYED_LAYERS
            built = _built(folders[dtype][name], dtype, need, max(need, 64))
            got[enabled] = run_plan_in_process(built.step_fn, plan)
            replayed = launch_memo.REPLAYED_LAYERS - before
            layers = TINY[name][0]["num_hidden_layers"]
            assert (replayed > 0) == (enabled and layers > 2), (what, enabled, replayed)
        assert got[True].keys() == got[False].keys()
        for step in got[True]:
            assert np.array_equal(got[True][step], got[False][step]), f"{name}/{dtype}/{what}: step {step} differs"


def test_pages_of_an_ended_request_are_cleared_before_reuse(tiny_folders_bf16):
    """A request ends and its pages are filled with NaN (as an overflow, or a step that gave up, could leave them);
    the next request gets those pages and its prompt ends in the middle of one. The prompt kernel that copies whole
    pages (head size 64) would multiply the stale slots by probabilities of zero: the logits must be finite and those
    of the plain implementation. The engine clears every page it hands out."""
    from dynalm_b200.engine import StepEntry, build
    name = "e"
    cfg = TINY[name][0]
    plain = PlainLlama(tiny_folders_bf16[name])
    built = build(tiny_folders_bf16[name], dtype="bfloat16", kv_tokens=192, max_batch_tokens=192, max_requests=2, context=256)
    first = random_requests(cfg["vocab_size"], [180], seed=50)["r0"]
    built.step_fn.step([StepEntry("a", first, [179])])
    built.step_fn.end("a")
    for g in built.cache.groups:
        g.storage.fill_(float("nan"))
    second = random_requests(cfg["vocab_size"], [150], seed=51)["r0"]
    got = built.step_fn.step([StepEntry("b", second[:137], [136])]).float().cpu().numpy()
    more = built.step_fn.step([StepEntry("b", second[137:], list(range(13)))]).float().cpu().numpy()
    want = plain.logits(second)
    assert np.isfinite(got).all() and np.isfinite(more).all()
    assert np.abs(got[0] - want[136]).max() <= TOL["bfloat16"][0]
    assert np.abs(more - want[137:]).max() <= TOL["bfloat16"][0]
    built.step_fn.end("b")
