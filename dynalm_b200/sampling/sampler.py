"""Per-request samplers.

Every request is sampled on the device (csrc/sampling.cu) from the logits rows of the step, and only token ids come
back: greedy, temperature, min-p, top-p and top-k up to 1,024 by kernels that need nothing from the host but a uniform
number; penalties by a kernel that gets the counts of the recent tokens from the host (and reads the token of a
step still in flight from the device). All of these can be decoded a step ahead. Top-k and top-p follow the reference's pipeline, penalties -> top-k -> temperature -> min-p -> top-p
-> draw (dynalm/src/sampling/sampler.cpp:96-220), by narrowing the vocabulary down to the places that pipeline turns
on. A row with top-k above 1,024 comes to the host, which runs the same pipeline here, as the reference does for
every request.
"""

from __future__ import annotations

from typing import Optional, Sequence

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

    DEVICE_TOP_K = 1024      # the candidates the filtered kernel keeps (SAMPLE_CAP in csrc/sampling.cu)

    @property
    def on_device(self) -> bool:
        """Whether the device can choose this request's token without the host's seeing the logits, so that the
        request can be decoded a step ahead: greedy, temperature, min-p, top-p, top-k up to DEVICE_TOP_K, and the
        penalties (the host counts the tokens it knows, the device adds the one in flight). A larger top-k needs
        the host to finish."""
        p = self.params
        return p.greedy or p.top_k <= self.DEVICE_TOP_K

    @property
    def wants_filtered(self) -> bool:
        """Top-k or top-p is set: the draw goes down the candidates in the order of their logits."""
        return self.params.top_k > 0 or self.params.top_p < 1.0

    @property
    def cut_offset(self) -> float:
        """min-p as an offset below the largest logit: temperature * log(min_p) (sampler.cpp:146); -inf when off."""
        p = self.params
        return float(p.temperature) * float(np.log(p.min_p)) if p.min_p > 0.0 and not p.greedy else -np.inf

    def next_uniform(self) -> float:
        return self.rng.uniform()

    def penalty_counts(self, context: Sequence[int], vocab: int, unseen: int = 0):
        """The distinct ids among the last `penalty_last_n` tokens of the context, and how often each occurs
        (what the penalties act on, sampler.cpp:96-116); two empty arrays where there is nothing to penalise.
        `unseen`: tokens that follow `context` and are not known here yet (a step in flight chose them); they take
        their places in the window, so that many fewer of `context` are counted."""
        p = self.params
        none = np.zeros(0, dtype=np.int64)
        if not p.has_penalties or len(context) + unseen == 0:
            return none, none
        n = len(context) + unseen if p.penalty_last_n < 0 else min(len(context) + unseen, p.penalty_last_n)
        n -= unseen
        if n <= 0:
            return none, none
        ids, counts = np.unique(np.asarray(context[len(context) - n:], dtype=np.int64), return_counts=True)
        ok = (ids >= 0) & (ids < vocab)
        return ids[ok], counts[ok]

    # ---- the host pipeline -----------------------------------------------------------------------
    def apply_penalties(self, logits: np.ndarray, context: Sequence[int]) -> None:
        """Repetition, frequency and presence penalties over the last `penalty_last_n` tokens
        (sampler.cpp:96-116). In place."""
        p = self.params
        ids, counts = self.penalty_counts(context, logits.size)
        if ids.size == 0:
            return
        l = logits[ids]
        if p.repetition_penalty != 1.0:
            l = np.where(l > 0, l / np.float32(p.repetition_penalty), l * np.float32(p.repetition_penalty))
        l = l - (counts.astype(np.float32) * np.float32(p.frequency_penalty) + np.float32(p.presence_penalty))
        logits[ids] = l

    def sample_host(self, logits: np.ndarray, context: Sequence[int], u: Optional[float] = None,
                    penalties_applied: bool = False) -> int:
        """The whole pipeline on one float32 logits row (which it may modify). `u`: the uniform number to draw
        with (one is taken from the request's generator otherwise); `penalties_applied`: the row has them already."""
        p = self.params
        if not penalties_applied:
            self.apply_penalties(logits, context)
        if p.greedy:
            return greedy_token(logits)
        vocab = logits.size
        max_l = float(logits.max())
        t = float(p.temperature)
        use_k = 0 < p.top_k < vocab
        if not use_k and p.top_p >= 1.0 and p.min_p <= 0.0:
            probs = np.exp((logits.astype(np.float64) - max_l) / t)
            return self._draw(np.arange(vocab), probs, float(probs.sum()), u)
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
        return self._draw(ids, probs, kept, u)

    def _draw(self, ids: np.ndarray, probs: np.ndarray, total: float, u: Optional[float] = None) -> int:
        """u * total walked down the candidates until it goes negative; the last one on rounding
        (sampler.cpp:209-220)."""
        u = (self.rng.uniform() if u is None else u) * total
        cum = np.cumsum(probs)
        i = int(np.searchsorted(cum, u, side="right"))
        return int(ids[min(i, ids.size - 1)])
