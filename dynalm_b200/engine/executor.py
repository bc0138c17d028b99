"""Runs the scheduler's batches on the GPU: the step function, then sampling on the device."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional

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
    completed its pending work. Greedy and temperature-only requests are sampled by kernels from
    the logits on the device and only their ids come back; requests with filters or penalties get
    their logits row on the host (see dynalm_b200.sampling.sampler).

    `launch(batch, after)` / `collect(launched)` split that in two for decode batches whose requests
    are all sampled on the device: the ids stay on the device, and a following batch can be launched
    `after` it, taking its tokens from those ids there, before the host has seen them."""

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
        if want and all(b.seq.sampler.on_device and b.seq.sampler.params.greedy for b in want):
            return (self._ids[:len(want)], self._ids[2 * self._n:])
        return None

    def _sample_on_device(self, logits: Optional[torch.Tensor], want: List[BatchItem], slot: int) -> None:
        n = len(want)
        if logits is None:
            # the step picked the most likely tokens itself (and brought the status word along)
            self._ids_host[slot].copy_(self._ids, non_blocking=True)
            self.d2h_bytes += self._ids_host[slot].numel() * 4
            return
        ops.argmax(logits, self._ids[:n], status_to=self._ids[2 * self._n:])
        if any(not b.seq.sampler.params.greedy and b.seq.sampler.on_device for b in want):
            th, uh = self._temp_host[slot], self._u_host[slot]
            for i, b in enumerate(want):
                p = b.seq.sampler.params
                on = not p.greedy and b.seq.sampler.on_device
                th[i] = p.temperature if on else 1.0
                uh[i] = b.seq.sampler.next_uniform() if on else 0.0
            self._temp[:n].copy_(th[:n], non_blocking=True)
            self._u[:n].copy_(uh[:n], non_blocking=True)
            self.h2d_bytes += 12 * n
            ops.sample_temperature(logits, self._temp, self._u, self._ids[self._n:self._n + n])
        self._ids_host[slot].copy_(self._ids, non_blocking=True)
        self.d2h_bytes += self._ids_host[slot].numel() * 4

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
        self._sample_on_device(logits, batch, slot)
        ev = torch.cuda.Event()
        ev.record()
        places = {b.seq.id: (i if b.seq.sampler.params.greedy else self._n + i) for i, b in enumerate(batch)}
        return Launched(places, slot, ev)

    def collect(self, launched: Launched) -> Dict[Hashable, int]:
        launched.event.synchronize()
        ids = self._ids_host[launched.slot].numpy()
        self._check_status(ids)
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
        if self.can_launch(batch):
            return self.collect(self.launch(batch))
        entries = [StepEntry(b.seq.id, b.tokens, [len(b.tokens) - 1] if b.sample else []) for b in batch]
        want = [b for b in batch if b.sample]
        logits = self.step_fn.step(entries, reserve=False, choose=self._choose(want))
        self.h2d_bytes += self.step_fn.batcher.last_upload_bytes
        if not want:
            return {}
        n = len(want)
        slot = self._turn
        self._turn ^= 1
        self._sample_on_device(logits, want, slot)
        host_rows = [(i, b) for i, b in enumerate(want) if not b.seq.sampler.on_device]
        rows = None
        if host_rows:
            idx = torch.tensor([i for i, _ in host_rows], device=logits.device)
            rows = logits[:n].index_select(0, idx).to("cpu", non_blocking=False).numpy()
            self.d2h_bytes += rows.nbytes
        torch.cuda.current_stream().synchronize()
        ids = self._ids_host[slot].numpy()
        self._check_status(ids)
        out: Dict[Hashable, int] = {}
        for i, b in enumerate(want):
            s = b.seq.sampler
            if s.on_device:
                out[b.seq.id] = int(ids[i] if s.params.greedy else ids[self._n + i])
        for k, (i, b) in enumerate(host_rows):
            # the context the penalties see: everything up to and including the tokens just computed
            out[b.seq.id] = b.seq.sampler.sample_host(rows[k], b.seq.tokens)
        return out
