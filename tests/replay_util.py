"""Replay plans for tests: ways of cutting the same requests into steps, and a comparer.

A plan is a list of steps in the format bin/trace_run reads, plus for every written logits row the
(request, position) it belongs to, so that all plans are compared with the same plain logits."""

from __future__ import annotations

import json
import os
import subprocess
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def random_requests(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = np.random.RandomState(seed)
    return {f"r{i}": [int(t) for t in rng.randint(0, vocab, size=n)] for i, n in enumerate(lengths)}


class Plan:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: Dict[int, List[Tuple[str, int]]] = {}     # step -> [(request, position)] in file order

    def add(self, entries: List[Tuple[str, List[int], int, List[int]]], end: Sequence[str] = ()):
        """entries: (request, tokens, start position, wanted places)."""
        step = len(self.steps)
        self.steps.append({"step": step, "entries": [{"id": r, "tokens": t, "want": w} for r, t, _, w in entries],
                           "end": list(end)})
        rows = [(r, s + i) for r, _, s, w in entries for i in w]
        if rows:
            self.rows[step] = rows
        return step

    def max_live_tokens(self, page: int = 64) -> int:
        """The most tokens live requests hold at any time, each rounded up to `page`."""
        held: Dict[str, int] = {}
        best = 0
        for st in self.steps:
            for e in st["entries"]:
                held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
            best = max(best, sum(-(-n // page) * page for n in held.values()))
            for r in st["end"]:
                held.pop(r, None)
        return best


def plan_whole(reqs: Dict[str, List[int]]) -> Plan:
    p = Plan()
    for r, toks in reqs.items():
        p.add([(r, toks, 0, list(range(len(toks))))], end=[r])
    return p


def plan_tail(reqs: Dict[str, List[int]], tail: int = 32) -> Plan:
    """Most of each request in one step, its last `tail` tokens one by one."""
    p = Plan()
    for r, toks in reqs.items():
        head = max(1, len(toks) - tail) if len(toks) > 1 else 1
        p.add([(r, toks[:head], 0, [head - 1])], end=[r] if head == len(toks) else [])
        for i in range(head, len(toks)):
            p.add([(r, [toks[i]], i, [0])], end=[r] if i == len(toks) - 1 else [])
    return p


def plan_chunks(reqs: Dict[str, List[int]], sizes: Sequence[int]) -> Plan:
    """Each request alone, in portions of changing size (down to two tokens), logits everywhere."""
    p = Plan()
    k = 0
    for r, toks in reqs.items():
        pos = 0
        while pos < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - pos)
            k += 1
            p.add([(r, toks[pos:pos + n], pos, list(range(n)))], end=[r] if pos + n == len(toks) else [])
            pos += n
    return p


def plan_mixed(reqs: Dict[str, List[int]], seed: int, max_live: int = 4, decode_tail: int = 8,
               sizes: Sequence[int] = (2, 3, 5, 7, 16, 24)) -> Plan:
    """Up to `max_live` requests alive: portions of some beside single tokens of others. A request
    is fed in random portions until `decode_tail` tokens remain, then one token a step; requests
    are sometimes left out of a step. Finished requests make room for waiting ones, so with a small
    pool their pages are used again."""
    rng = np.random.RandomState(seed)
    p = Plan()
    waiting = list(reqs)
    live: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for r in list(live):
            toks, pos = reqs[r], live[r]
            if len(live) > 1 and rng.rand() < 0.2:
                continue                                   # left out of this step
            left = len(toks) - pos
            n = 1 if left <= decode_tail else int(min(sizes[rng.randint(len(sizes))], left - decode_tail))
            want = list(range(n)) if n == 1 or rng.rand() < 0.7 else [n - 1]
            entries.append((r, toks[pos:pos + n], pos, want))
            live[r] = pos + n
            if live[r] == len(toks):
                ended.append(r)
        if not entries:
            continue
        order = rng.permutation(len(entries))
        p.add([entries[i] for i in order], end=ended)
        for r in ended:
            del live[r]
    return p


def plan_many_rows(short: Dict[str, List[int]], long: Dict[str, List[int]], seed: int, tail_lo: int = 10,
                   tail_hi: int = 22, sizes: Sequence[int] = (9, 2, 21, 5, 33)) -> Plan:
    """Many live requests: the `short` ones (17 to 40 of them) are first brought in, four prompts a step; then every
    step carries one token of each short request that has tokens left, beside a portion of one of the `long`
    requests while there is one, and alone afterwards. The short requests end at different times, so the number of
    single-token rows falls step by step from len(short); logits are wanted at every single-token row and at the
    end of every portion."""
    rng = np.random.RandomState(seed)
    p = Plan()
    names = list(short)
    tails = {r: int(min(len(short[r]) - 1, rng.randint(tail_lo, tail_hi + 1))) for r in names}
    for i in range(0, len(names), 4):
        group = names[i:i + 4]
        p.add([(r, short[r][:len(short[r]) - tails[r]], 0, [len(short[r]) - tails[r] - 1]) for r in group])
    done = {r: len(short[r]) - tails[r] for r in names}
    waiting = list(long)
    cur, cur_pos, k = None, 0, 0
    while any(done[r] < len(short[r]) for r in names) or waiting or cur is not None:
        entries, ended = [], []
        for r in names:
            if done[r] < len(short[r]):
                entries.append((r, [short[r][done[r]]], done[r], [0]))
                done[r] += 1
                if done[r] == len(short[r]):
                    ended.append(r)
        if cur is None and waiting:
            cur, cur_pos = waiting.pop(0), 0
        if cur is not None:
            toks = long[cur]
            n = min(sizes[k % len(sizes)], len(toks) - cur_pos)
            k += 1
            entries.append((cur, toks[cur_pos:cur_pos + n], cur_pos, [n - 1]))
            cur_pos += n
            if cur_pos == len(toks):
                ended.append(cur)
                cur = None
        p.add(entries, end=ended)
    return p


def kl_and_top1(plan: Plan, got: Dict[int, np.ndarray], plain: Dict[str, np.ndarray], near_tie: float = 0.0):
    """Over all written rows: the mean KL divergence from the plain distribution to the one got, and the share of
    rows whose largest logit is at the same token (rows whose two largest plain logits lie within `near_tie` of each
    other count as agreeing)."""
    kls, same = [], []
    for step in sorted(plan.rows):
        for i, (r, pos) in enumerate(plan.rows[step]):
            ref = plain[r][pos].astype(np.float64)
            g = got[step][i].astype(np.float64)
            lp_ref = ref - ref.max() - np.log(np.exp(ref - ref.max()).sum())
            lp_got = g - g.max() - np.log(np.exp(g - g.max()).sum())
            kls.append(float((np.exp(lp_ref) * (lp_ref - lp_got)).sum()))
            top = np.sort(ref)[-2:]
            same.append(bool(ref.argmax() == g.argmax()) or (top[1] - top[0]) <= near_tie)
    return float(np.mean(kls)), float(np.mean(same))


def run_plan_in_process(step_fn, plan: Plan) -> Dict[int, np.ndarray]:
    from dynalm_b200.engine import StepEntry
    out = {}
    for st in plan.steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]]
        logits = step_fn.step(entries)
        if logits is not None:
            out[st["step"]] = logits.float().cpu().numpy().copy()
        for r in st["end"]:
            step_fn.end(r)
        step_fn.cache.check()
    assert not step_fn.live(), "a plan must end every request it starts"
    return out


def run_plan_trace_run(model_dir: str, dtype: str, plan: Plan, out_dir: str, max_tokens: int, vocab: int,
                       env=None, summary: str = None) -> Dict[int, np.ndarray]:
    """Through bin/trace_run as a user would: one process, steps on stdin, files out."""
    text = "".join(json.dumps(s) + "\n" for s in plan.steps)
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out",
                           out_dir, "--max-tokens", str(max_tokens)] + (["--summary", summary] if summary else []),
                          input=text, capture_output=True, text=True, env=env, timeout=900)
    assert proc.returncode == 0, f"trace_run failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in plan.steps]
    out = {}
    for step in plan.rows:
        out[step] = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(-1, vocab)
    return out


def compare(plan: Plan, got: Dict[int, np.ndarray], plain: Dict[str, np.ndarray], tol_abs: float, tol_rel: float,
            what: str) -> float:
    """Every written row against the plain logits of its (request, position). Names the first bad
    row: its request, position and step."""
    worst = 0.0
    assert set(got) == set(plan.rows), f"{what}: steps with output {sorted(got)} != expected {sorted(plan.rows)}"
    for step in sorted(plan.rows):
        rows = plan.rows[step]
        assert got[step].shape[0] == len(rows), f"{what}: step {step} wrote {got[step].shape[0]} rows, wanted {len(rows)}"
        for i, (r, pos) in enumerate(rows):
            ref = plain[r][pos]
            err = float(np.abs(got[step][i] - ref).max())
            bound = tol_abs + tol_rel * float(np.abs(ref).max())
            assert err <= bound, (f"{what}: first wrong row is step {step}, request {r}, position {pos}: "
                                  f"max |diff| {err:.3g} > {bound:.3g}")
            worst = max(worst, err)
    return worst
