"""Per-request samplers.

Greedy and temperature-only requests are sampled on the device (csrc/sampling.cu) from the logits
rows of the step; only token ids come back. Requests with top-k / top-p / min-p or penalties take
the reference's full pipeline, penalties -> top-k -> temperature -> min-p -> top-p -> draw
(dynalm/src/sampling/sampler.cpp:96-220), on the host from their one logits row, as the reference
does for every request.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np

from .params import SamplingParams
from .rng import Xoshiro256


def greedy_token(logits: np.ndarray) -> int:
    """Index of the largest logit, the lowest id among ties (sampler.cpp:31-38)."""
    if logits.size == 0:
        return 0
    best = logits.max()
    hits = np.flatnonzero(logits == best)
    return int(hits[0]) if hits.size else 0


class Sampler:
    """One request's sampling state: its parameters and its own generator."""

    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params
        self.rng = Xoshiro256(params.seed)

    @property
    def on_device(self) -> bool:
        p = self.params
        return not p.has_penalties and (p.greedy or not p.has_filters)

    def next_uniform(self) -> float:
        return self.rng.uniform()

    # ---- the host pipeline -----------------------------------------------------------------------
    def apply_penalties(self, logits: np.ndarray, context: Sequence[int]) -> None:
        """Repetition, frequency and presence penalties over the last `penalty_last_n` tokens
        (sampler.cpp:96-116). In place."""
        p = self.params
        if not p.has_penalties or len(context) == 0:
            return
        n = len(context) if p.penalty_last_n < 0 else min(len(context), p.penalty_last_n)
        if n == 0:
            return
        ids, counts = np.unique(np.asarray(context[len(context) - n:], dtype=np.int64), return_counts=True)
        ok = (ids >= 0) & (ids < logits.size)
        ids, counts = ids[ok], counts[ok]
        l = logits[ids]
        if p.repetition_penalty != 1.0:
            l = np.where(l > 0, l / np.float32(p.repetition_penalty), l * np.float32(p.repetition_penalty))
        l = l - (counts.astype(np.float32) * np.float32(p.frequency_penalty) + np.float32(p.presence_penalty))
        logits[ids] = l

    def sample_host(self, logits: np.ndarray, context: Sequence[int]) -> int:
        """The whole pipeline on one float32 logits row (which it may modify)."""
        p = self.params
        self.apply_penalties(logits, context)
        if p.greedy:
            return greedy_token(logits)
        vocab = logits.size
        max_l = float(logits.max())
        t = float(p.temperature)
        use_k = 0 < p.top_k < vocab
        if not use_k and p.top_p >= 1.0 and p.min_p <= 0.0:
            probs = np.exp((logits.astype(np.float64) - max_l) / t)
            return self._draw(np.arange(vocab), probs, float(probs.sum()))
        # min-p: keep logits within T * log(min_p) of the maximum (sampler.cpp:146)
        cut = max_l + t * np.log(p.min_p) if p.min_p > 0.0 else -np.inf
        ids = np.flatnonzero(logits >= cut)
        if ids.size == 0:
            return greedy_token(logits)
        cand = logits[ids].astype(np.float64)
        total = float(np.exp((cand - max_l) / t).sum())          # mass after min-p
        if use_k or p.top_p < 1.0:
            order = np.lexsort((ids, -cand))                     # logit descending, id ascending
            ids, cand = ids[order], cand[order]
            if use_k:
                ids, cand = ids[:p.top_k], cand[:p.top_k]
        probs = np.exp((cand - max_l) / t)
        kept = float(probs.sum())
        if p.top_p < 1.0:
            # nucleus over the distribution after top-k / min-p (sampler.cpp:196-205)
            target = p.top_p * (kept if use_k else total)
            cum = np.cumsum(probs)
            keep = int(np.searchsorted(cum, target, side="left")) + 1
            keep = max(1, min(keep, probs.size))
            ids, probs = ids[:keep], probs[:keep]
            kept = float(probs.sum())
        return self._draw(ids, probs, kept)

    def _draw(self, ids: np.ndarray, probs: np.ndarray, total: float) -> int:
        """u * total walked down the candidates until it goes negative; the last one on rounding
        (sampler.cpp:209-220)."""
        u = self.rng.uniform() * total
        cum = np.cumsum(probs)
        i = int(np.searchsorted(cum, u, side="right"))
        return int(ids[min(i, ids.size - 1)])
