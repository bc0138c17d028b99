"""Sampling on the CPU: parameters, the generator, and the host pipeline (penalties -> top-k ->
temperature -> min-p -> top-p -> draw) against a straightforward restatement of the reference's
rules (dynalm/src/sampling/sampler.cpp:31-220)."""

import math

import numpy as np
import pytest

from dynalm_b200.errors import InvalidArgument
from dynalm_b200.sampling import Sampler, SamplingParams, Xoshiro256, greedy_token
from plain_llama import Xoshiro256 as PlainRng
from plain_llama import sample_temperature


def test_params_ranges():
    SamplingParams().validate()
    for bad in (dict(temperature=-0.1), dict(temperature=101.0), dict(top_k=-1), dict(top_p=0.0), dict(top_p=1.5),
                dict(min_p=-0.1), dict(min_p=1.1), dict(repetition_penalty=0.0), dict(frequency_penalty=2.5),
                dict(presence_penalty=-2.5), dict(penalty_last_n=-2), dict(temperature=float("nan"))):
        with pytest.raises(InvalidArgument):
            SamplingParams(**bad).validate()
    assert SamplingParams().greedy and SamplingParams(temperature=0.7, top_k=1).greedy
    assert not SamplingParams(temperature=0.7).greedy and SamplingParams(presence_penalty=0.5).has_penalties


def test_generator_matches_the_plain_one_and_is_uniform():
    a, b = Xoshiro256(1234), PlainRng(1234)
    assert [a.next() for _ in range(50)] == [b.next() for _ in range(50)]
    assert Xoshiro256(1).next() != Xoshiro256(2).next()
    u = np.array([Xoshiro256(7).uniform()] + [a.uniform() for _ in range(20000)])
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.01


def test_greedy_ties_go_to_the_lowest_id():
    assert greedy_token(np.array([1.0, 3.0, 3.0, 2.0], dtype=np.float32)) == 1
    assert greedy_token(np.array([], dtype=np.float32)) == 0
    s = Sampler(SamplingParams())
    assert s.on_device and s.sample_host(np.array([0.1, 0.9, 0.9], dtype=np.float32), []) == 1


def test_temperature_only_follows_the_walk():
    rng = np.random.RandomState(0)
    logits = (rng.randn(500) * 2).astype(np.float32)
    s = Sampler(SamplingParams(temperature=0.8, seed=5))
    ref_rng = PlainRng(5)
    for _ in range(200):
        assert s.sample_host(logits.copy(), []) == sample_temperature(logits, 0.8, ref_rng.uniform())


def _support(params, logits, draws=4000):
    s = Sampler(params)
    return {s.sample_host(logits.copy(), []) for _ in range(draws)}


def test_filters_keep_the_right_support():
    logits = np.log(np.array([0.4, 0.25, 0.15, 0.1, 0.05, 0.03, 0.02], dtype=np.float64)).astype(np.float32)
    assert _support(SamplingParams(temperature=1.0, top_k=3, seed=1), logits) == {0, 1, 2}
    # nucleus 0.7: 0.4 + 0.25 = 0.65 < 0.7, the third token completes it
    assert _support(SamplingParams(temperature=1.0, top_p=0.7, seed=2), logits) == {0, 1, 2}
    # min-p 0.2: keep p >= 0.2 * 0.4 = 0.08
    assert _support(SamplingParams(temperature=1.0, min_p=0.2, seed=3), logits) == {0, 1, 2, 3}
    # with top-k the nucleus applies to what top-k kept: 0.9 of (0.4 + 0.25 + 0.15) = 0.72 -> all three
    assert _support(SamplingParams(temperature=1.0, top_k=3, top_p=0.9, seed=4), logits) == {0, 1, 2}
    assert _support(SamplingParams(temperature=1.0, top_k=3, top_p=0.5, seed=4), logits) == {0, 1}


def test_temperature_ratio():
    """P(a)/P(b) = (pa/pb)^(1/T) (the reference's own check, dynalm/tests/test_engine.cpp:507-680)."""
    logits = np.log(np.array([0.5, 0.3, 0.2])).astype(np.float32)
    T = 0.5
    s = Sampler(SamplingParams(temperature=T, seed=11))
    counts = np.bincount([s.sample_host(logits.copy(), []) for _ in range(20000)], minlength=3)
    assert abs(counts[0] / counts[1] - (0.5 / 0.3) ** (1 / T)) < 0.25


def test_penalties_arithmetic():
    logits = np.array([2.0, -1.0, 0.5, 3.0], dtype=np.float32)
    s = Sampler(SamplingParams(repetition_penalty=2.0, frequency_penalty=0.5, presence_penalty=0.25, penalty_last_n=3))
    out = logits.copy()
    s.apply_penalties(out, [3, 0, 1, 1, 0])          # the last three: 1, 1, 0
    assert out[3] == 3.0 and out[2] == 0.5            # outside the window / absent
    assert math.isclose(out[0], 2.0 / 2.0 - (1 * 0.5 + 0.25), rel_tol=1e-6)
    assert math.isclose(out[1], -1.0 * 2.0 - (2 * 0.5 + 0.25), rel_tol=1e-6)
    assert s.on_device            # penalties do not keep a request from being decoded a step ahead
    assert not Sampler(SamplingParams(temperature=0.8, top_k=5000)).on_device     # a top-k that the kernel leaves to the host
    # a token still in flight takes its place in the window: the last three are then 1, 0 and the unseen one
    ids, counts = s.penalty_counts([3, 0, 1, 1, 0], 4, unseen=1)
    assert ids.tolist() == [0, 1] and counts.tolist() == [1, 1]
    whole = Sampler(SamplingParams(presence_penalty=1.0, penalty_last_n=-1))
    out = logits.copy()
    whole.apply_penalties(out, [3, 0, 1, 1, 0])
    assert out.tolist() == [1.0, -2.0, 0.5, 2.0]


def test_same_seed_repeats_other_seed_differs():
    logits = (np.random.RandomState(1).randn(300)).astype(np.float32)
    p = dict(temperature=0.9, top_k=40, top_p=0.95)
    a = [Sampler(SamplingParams(seed=3, **p)).sample_host(logits.copy(), []) for _ in range(1)]
    run = lambda seed: (lambda s: [s.sample_host(logits.copy(), []) for _ in range(30)])(Sampler(SamplingParams(seed=seed, **p)))
    assert run(3) == run(3) and run(3) != run(4)
