"""Runs the scheduler's batches on the GPU: the step function, then sampling on the device."""

from __future__ import annotations

from typing import Dict, Hashable, List

import numpy as np
import torch

from ..errors import EngineError
from ..kernels import ops
from .scheduler import BatchItem
from .step import StepEntry, StepFunction


class GpuExecutor:
    """`run(batch)`: one step of the model for the whole batch, then one token for every item that
    completed its pending work. Greedy and temperature-only requests are sampled by kernels from
    the logits on the device and only their ids come back; requests with filters or penalties get
    their logits row on the host (see dynalm_b200.sampling.sampler)."""

    def __init__(self, step_fn: StepFunction):
        self.step_fn = step_fn
        self.cache = step_fn.cache
        self.max_tokens = step_fn.max_tokens
        self.vocab = step_fn.vocab
        dev = step_fn.rt.device
        n = step_fn.max_requests
        self._ids = torch.zeros(2 * n, dtype=torch.int32, device=dev)            # greedy | drawn
        self._ids_host = torch.zeros(2 * n, dtype=torch.int32).pin_memory()
        self._temp_host = torch.ones(n, dtype=torch.float32).pin_memory()
        self._u_host = torch.zeros(n, dtype=torch.float64).pin_memory()
        self._temp = torch.ones(n, dtype=torch.float32, device=dev)
        self._u = torch.zeros(n, dtype=torch.float64, device=dev)
        self.h2d_bytes = 0
        self.steps = 0
        self.d2h_bytes = 0

    def begin(self, request_id: Hashable) -> None:
        self.step_fn.begin(request_id)

    def end(self, request_id: Hashable) -> None:
        self.step_fn.end(request_id)

    def run(self, batch: List[BatchItem]) -> Dict[Hashable, int]:
        entries = [StepEntry(b.seq.id, b.tokens, [len(b.tokens) - 1] if b.sample else []) for b in batch]
        logits = self.step_fn.step(entries, reserve=False)
        self.h2d_bytes += self.step_fn.buffers.size * 4
        want = [b for b in batch if b.sample]
        if not want:
            return {}
        n = len(want)
        max_n = self._temp_host.numel()
        drawn = any(not b.seq.sampler.params.greedy and b.seq.sampler.on_device for b in want)
        ops.argmax(logits, self._ids[:n])
        if drawn:
            for i, b in enumerate(want):
                p = b.seq.sampler.params
                on = not p.greedy and b.seq.sampler.on_device
                self._temp_host[i] = p.temperature if on else 1.0
                self._u_host[i] = b.seq.sampler.next_uniform() if on else 0.0
            self._temp[:n].copy_(self._temp_host[:n], non_blocking=True)
            self._u[:n].copy_(self._u_host[:n], non_blocking=True)
            self.h2d_bytes += 12 * n
            ops.sample_temperature(logits, self._temp, self._u, self._ids[max_n:max_n + n])
        self._ids_host.copy_(self._ids, non_blocking=True)
        host_rows = [(i, b) for i, b in enumerate(want) if not b.seq.sampler.on_device]
        rows = None
        if host_rows:
            idx = torch.tensor([i for i, _ in host_rows], device=logits.device)
            rows = logits[:n].index_select(0, idx).to("cpu", non_blocking=False).numpy()
            self.d2h_bytes += rows.nbytes
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += self._ids_host.numel() * 4
        self.steps += 1
        if self.steps % 64 == 1 and ops.gemm_tcgen05_status() != 0:
            raise EngineError("a tcgen05 matrix product gave up waiting on a barrier; its results are not valid")
        ids = self._ids_host.numpy()
        out: Dict[Hashable, int] = {}
        for i, b in enumerate(want):
            s = b.seq.sampler
            if s.on_device:
                out[b.seq.id] = int(ids[i] if s.params.greedy else ids[max_n + i])
        for k, (i, b) in enumerate(host_rows):
            # the context the penalties see: everything up to and including the tokens just computed
            out[b.seq.id] = b.seq.sampler.sample_host(rows[k], b.seq.tokens)
        return out
