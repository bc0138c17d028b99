"""Runs the scheduler's batches on the GPU: the step function, then sampling on the device."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional

import numpy as np
import torch

from ..errors import EngineError
from ..kernels import ops
from .scheduler import BatchItem
from .step import StepEntry, StepFunction


@dataclass
class Launched:
    """A batch that has been issued to the GPU and whose chosen ids are on their way to the host."""

    places: Dict[Hashable, int]        # request -> place of its chosen id in the ids buffer
    slot: int                          # which pinned host copy receives the ids
    event: torch.cuda.Event


class GpuExecutor:
    """`run(batch)`: one step of the model for the whole batch, then one token for every item that
    completed its pending work. Every request is sampled by kernels from the logits on the device and only the ids
    come back; a row of a request with top-k or top-p whose candidates do not fit the kernel gets its logits on the
    host (see dynalm_b200.sampling.sampler).

    `launch(batch, after)` / `collect(launched)` split that in two for decode batches whose requests
    are all sampled on the device: the ids stay on the device, and a following batch can be launched
    `after` it, taking its tokens from those ids there, before the host has seen them."""

    PENALTY_TRIPLES = 1 << 16      # distinct recent tokens over all penalised rows of a step

    def __init__(self, step_fn: StepFunction):
        self.step_fn = step_fn
        self.cache = step_fn.cache
        self.max_tokens = step_fn.max_tokens
        self.vocab = step_fn.vocab
        dev = step_fn.rt.device
        n = step_fn.max_requests
        self._n = n
        # greedy | drawn | the device's status word as the step left it (a code when a bounded wait inside a kernel
        # gave up): it reaches the host in the copy of the ids, so every step is checked without another wait
        self._ids = torch.zeros(2 * n + 1, dtype=torch.int32, device=dev)
        # two host copies of everything a launch leaves behind: one launch may be in flight while the next is made
        self._ids_host = [torch.zeros(2 * n + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._temp_host = [torch.ones(n, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._u_host = [torch.zeros(n, dtype=torch.float64).pin_memory() for _ in range(2)]
        self._temp = torch.ones(n, dtype=torch.float32, device=dev)
        self._u = torch.zeros(n, dtype=torch.float64, device=dev)
        # What penalties and filters need from the host, two pinned copies of each as above, sent in one copy of
        # integers and one of doubles. Integers, by name -> (first element, elements): the rows with penalties, the
        # rows of the filtered kernel, their top-k, the penalties' (repetition, frequency, presence) as float32 bits,
        # where each penalised row's triples begin, the place among the ids of the token a step in flight chose for
        # it (or -1), and the triples (selection, id, count). Doubles: the filtered kernel's (temperature, min-p
        # offset, top-p, uniform) and the walk's min-p offsets.
        self._int_at = {}
        at = 0
        for name, count in (("penalised_rows", n), ("filtered_rows", n), ("top_k", n), ("penalty_params", 3 * n),
                            ("first_triple", n + 1), ("pending", n), ("triples", 3 * self.PENALTY_TRIPLES)):
            self._int_at[name] = (at, count)
            at += count
        self._dbl_at = {"filtered_params": (0, 4 * n), "cut_offsets": (4 * n, n)}
        self._stage_i = torch.zeros(at, dtype=torch.int32, device=dev)
        self._stage_d = torch.zeros(5 * n, dtype=torch.float64, device=dev)
        self._stage_i_host = [torch.zeros(self._stage_i.numel(), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._stage_d_host = [torch.zeros(self._stage_d.numel(), dtype=torch.float64).pin_memory() for _ in range(2)]
        self.host_sampled = 0      # rows that the filtered kernel left to the host so far
        self._turn = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.steps = 0

    def begin(self, request_id: Hashable) -> None:
        self.step_fn.begin(request_id)

    def end(self, request_id: Hashable) -> None:
        self.step_fn.end(request_id)

    # ---- device-sampled batches: launch now, collect later -------------------------------------------
    @staticmethod
    def can_launch(batch: List[BatchItem]) -> bool:
        return bool(batch) and all(b.sample and len(b.tokens) == 1 and b.seq.sampler.on_device for b in batch)

    def _choose(self, want: List[BatchItem]):
        """What to hand the step as `choose` when every wanted row is decided by its largest logit on the device."""
        if want and all(b.seq.sampler.params.greedy and not b.seq.sampler.params.has_penalties for b in want):
            return (self._ids[:len(want)], self._ids[2 * self._n:])
        return None

    def _ints(self, name: str, count: Optional[int] = None, host=None):
        """The named stretch of the staged integers (its first `count` elements): on the device, or of the host copy
        `host` (a NumPy view)."""
        at, most = self._int_at[name]
        count = most if count is None else count
        return (self._stage_i if host is None else host)[at:at + count]

    def _doubles(self, name: str, count: Optional[int] = None, host=None):
        at, most = self._dbl_at[name]
        count = most if count is None else count
        return (self._stage_d if host is None else host)[at:at + count]

    def _stage_penalties(self, ints, want: List[BatchItem], penalised: List[int], after: Optional[Launched]) -> int:
        """Writes what the penalties kernel needs for the rows `penalised` into the host copy `ints`; returns the
        number of triples. The context the penalties see: everything up to and including the tokens just computed."""
        n_triples, found = 0, []
        params = self._ints("penalty_params", host=ints).view(np.float32)
        first, pending = self._ints("first_triple", host=ints), self._ints("pending", host=ints)
        for j, i in enumerate(penalised):
            sampler, seq = want[i].seq.sampler, want[i].seq
            p = sampler.params
            unseen = 1 if after is not None and seq.id in after.places else 0
            ids, counts = sampler.penalty_counts(seq.tokens, self.vocab, unseen=unseen)
            params[3 * j:3 * j + 3] = (p.repetition_penalty, p.frequency_penalty, p.presence_penalty)
            first[j] = n_triples
            pending[j] = after.places[seq.id] if unseen and p.penalty_last_n != 0 else -1
            if ids.size:
                found.append(np.stack([np.full(ids.size, j, dtype=np.int64), ids, counts], axis=1))
                n_triples += ids.size
        first[len(penalised)] = n_triples
        self._ints("penalised_rows", len(penalised), host=ints)[:] = penalised
        if n_triples > self.PENALTY_TRIPLES:
            raise EngineError(f"penalties over {n_triples} distinct recent tokens in one step; the executor has room "
                              f"for {self.PENALTY_TRIPLES}")
        if found:
            self._ints("triples", 3 * n_triples, host=ints)[:] = np.concatenate(found).astype(np.int32).ravel()
        return n_triples

    def _sample_on_device(self, logits: Optional[torch.Tensor], want: List[BatchItem], slot: int,
                          after: Optional[Launched] = None) -> Dict[int, float]:
        """Choose a token for every wanted row on the device and start the copy of the ids to the host: the largest
        logit for every row (place i), and for the rows that draw, a draw (place n + i): a walk down the ids for
        temperature and min-p, the filtered kernel for top-k and top-p, which may leave -1 for the host to finish.
        Rows with penalties have them applied to their logits first; with `after`, the token that launch chose for
        the request is in no context yet, and the penalties kernel counts it from the ids on the device. Returns
        row -> the uniform number it drew with, for the rows of the filtered kernel."""
        n = len(want)
        if logits is None:
            # the step picked the most likely tokens itself (and brought the status word along)
            self._ids_host[slot].copy_(self._ids, non_blocking=True)
            self.d2h_bytes += self._ids_host[slot].numel() * 4
            return {}
        samplers = [b.seq.sampler for b in want]
        # top-k of the whole vocabulary or more is no filter (sampler.cpp:118): such a draw walks the ids in their order
        sorted_draw = [not s.params.greedy and (0 < s.params.top_k < self.vocab or s.params.top_p < 1.0) for s in samplers]
        penalised = [i for i, s in enumerate(samplers) if s.params.has_penalties]
        filtered = [i for i in range(n) if sorted_draw[i]]
        walk = [i for i, s in enumerate(samplers) if not s.params.greedy and not sorted_draw[i]]
        with_cut = any(samplers[i].params.min_p > 0.0 for i in walk)
        drawn: Dict[int, float] = {}

        # ---- what the kernels need from the host: two copies from pinned memory, integers and doubles ----
        ints, dbls = self._stage_i_host[slot].numpy(), self._stage_d_host[slot].numpy()
        n_triples = self._stage_penalties(ints, want, penalised, after) if penalised else 0
        if filtered:
            self._ints("filtered_rows", len(filtered), host=ints)[:] = filtered
            self._ints("top_k", len(filtered), host=ints)[:] = [samplers[i].params.top_k for i in filtered]
            params = self._doubles("filtered_params", host=dbls)
            for j, i in enumerate(filtered):
                p = samplers[i].params
                drawn[i] = samplers[i].next_uniform()
                params[4 * j:4 * j + 4] = (p.temperature, samplers[i].cut_offset, p.top_p, drawn[i])
        if with_cut:
            cuts = self._doubles("cut_offsets", n, host=dbls)
            cuts[:] = -np.inf
            for i in walk:
                cuts[i] = samplers[i].cut_offset
        if penalised or filtered:
            used = self._int_at["triples"][0] + 3 * n_triples
            self._stage_i[:used].copy_(self._stage_i_host[slot][:used], non_blocking=True)
            self.h2d_bytes += 4 * used
        if filtered or with_cut:
            used = self._dbl_at["cut_offsets"][0] + (n if with_cut else 0)
            self._stage_d[:used].copy_(self._stage_d_host[slot][:used], non_blocking=True)
            self.h2d_bytes += 8 * used

        # ---- the kernels, in the pipeline's order ----
        if penalised:
            ahead = after is not None
            ops.apply_penalties(logits, self._ints("penalised_rows", len(penalised)), self._ints("triples", 3 * n_triples),
                                n_triples, self._ints("penalty_params", 3 * len(penalised)).view(torch.float32),
                                self._ints("first_triple", len(penalised) + 1), chosen=self._ids if ahead else None,
                                pending=self._ints("pending", len(penalised)) if ahead else None)
        ops.argmax(logits, self._ids[:n], status_to=self._ids[2 * self._n:])
        if walk:
            th, uh = self._temp_host[slot], self._u_host[slot]
            th[:n] = 1.0
            uh[:n] = 0.0
            for i in walk:
                th[i] = samplers[i].params.temperature
                uh[i] = samplers[i].next_uniform()
            self._temp[:n].copy_(th[:n], non_blocking=True)
            self._u[:n].copy_(uh[:n], non_blocking=True)
            self.h2d_bytes += 12 * n
            ops.sample_temperature(logits, self._temp, self._u, self._ids[self._n:self._n + n],
                                   cut_offset=self._doubles("cut_offsets", n) if with_cut else None)
        if filtered:
            ops.sample_filtered(logits, self._ints("filtered_rows", len(filtered)), len(filtered),
                                self._doubles("filtered_params", 4 * len(filtered)), self._ints("top_k", len(filtered)),
                                self._ids[self._n:self._n + n])
        self._ids_host[slot].copy_(self._ids, non_blocking=True)
        self.d2h_bytes += self._ids_host[slot].numel() * 4
        return drawn

    def launch(self, batch: List[BatchItem], after: Optional[Launched] = None) -> Launched:
        """Issue a decode batch whose requests are all sampled on the device. With `after`, every request of the
        batch takes its token on the device from what `after` chose for it."""
        entries = [StepEntry(b.seq.id, b.tokens, [0]) for b in batch]
        feedback = None
        if after is not None:
            feedback = (self._ids, [after.places[b.seq.id] for b in batch])
        logits = self.step_fn.step(entries, reserve=False, token_feedback=feedback, choose=self._choose(batch))
        self.h2d_bytes += self.step_fn.batcher.last_upload_bytes
        slot = self._turn
        self._turn ^= 1
        self._sample_on_device(logits, batch, slot, after=after)
        ev = torch.cuda.Event()
        ev.record()
        places = {b.seq.id: (i if b.seq.sampler.params.greedy else self._n + i) for i, b in enumerate(batch)}
        return Launched(places, slot, ev)

    def collect(self, launched: Launched) -> Dict[Hashable, int]:
        launched.event.synchronize()
        ids = self._ids_host[launched.slot].numpy()
        self._check_status(ids)
        # (a negative id: the filtered kernel gave up on the row, whose largest logit is not finite or whose range is
        # so wide that bins of it still hold different logits; its logits are gone by now, the next step being in
        # flight, and the scheduler fails that request alone)
        return {req: int(ids[place]) for req, place in launched.places.items()}

    def _check_status(self, ids) -> None:
        """`ids`: the host copy of a step's chosen ids, whose last element is the status word as that step left it.
        A code there means that a kernel of the step (or of a step launched since the last check) gave up a bounded
        wait: nothing those steps computed is valid, keys and values they wrote included. The word is cleared, so
        that the steps after the failed requests have been dropped start clean."""
        self.steps += 1
        code = int(ids[2 * self._n])
        if code != 0:
            ops.clear_status(self.step_fn.rt.device)
            raise EngineError(f"a kernel gave up waiting on a barrier (status {code}); the step's results are not valid")

    # ---- any batch, synchronously ------------------------------------------------------------------------
    def run(self, batch: List[BatchItem]) -> Dict[Hashable, int]:
        if self.can_launch(batch) and not any(b.seq.sampler.wants_filtered and not b.seq.sampler.params.greedy for b in batch):
            return self.collect(self.launch(batch))
        # (with the logits still at hand a row that the filtered kernel leaves undecided can be finished on the host)
        entries = [StepEntry(b.seq.id, b.tokens, [len(b.tokens) - 1] if b.sample else []) for b in batch]
        want = [b for b in batch if b.sample]
        logits = self.step_fn.step(entries, reserve=False, choose=self._choose(want))
        self.h2d_bytes += self.step_fn.batcher.last_upload_bytes
        if not want:
            return {}
        n = len(want)
        slot = self._turn
        self._turn ^= 1
        drawn = self._sample_on_device(logits, want, slot)
        torch.cuda.current_stream().synchronize()
        ids = self._ids_host[slot].numpy()
        self._check_status(ids)
        out: Dict[Hashable, int] = {}
        host_rows = []
        for i, b in enumerate(want):
            token = int(ids[i] if b.seq.sampler.params.greedy else ids[self._n + i])
            if token == ops.SAMPLE_FILTERED_HOST:
                host_rows.append((i, b))
            else:
                out[b.seq.id] = token
        if host_rows:
            # rows whose candidates did not fit the filtered kernel: the same pipeline on the host, from the row's
            # logits (which have their penalties already) and with the uniform number the kernel was given
            idx = torch.tensor([i for i, _ in host_rows], device=logits.device)
            rows = logits[:n].index_select(0, idx).to("cpu", non_blocking=False).numpy()
            self.d2h_bytes += rows.nbytes
            self.host_sampled += len(host_rows)
            for k, (i, b) in enumerate(host_rows):
                out[b.seq.id] = b.seq.sampler.sample_host(rows[k], b.seq.tokens, u=drawn[i], penalties_applied=True)
        return out
