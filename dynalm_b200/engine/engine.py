"""The programmatic entry point: `Engine(model).generate(prompts)`.

The reference's entry is C++ (`Engine::create(EngineOptions)`, `generate_text`, `RequestStream`,
dynalm/src/runtime/engine.h:59-104,176-225,292-337) and starts at text; this engine starts at
token ids, so prompts are lists of ids and results are lists of ids. Option names follow
`EngineOptions` / `dynalm run`: `ctx` is the KV capacity in tokens, `batch` the most tokens per
forward pass.
"""

from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence, Union

import torch

from ..cache import DEFAULT_PAGE_SIZE
from ..errors import InvalidArgument
from ..sampling import SamplingParams
from .build import BuiltModel, build
from .executor import GpuExecutor
from .scheduler import Event, Request, Scheduler, SchedulerConfig
from .step import StepEntry


@dataclass
class Generation:
    """One finished request."""

    tokens: List[int]
    finish_reason: Optional[str]
    status: str
    error: Optional[str]
    prompt_tokens: int
    ttft_ms: float = 0.0
    total_ms: float = 0.0


class RequestStream:
    """The events of one request, for a thread other than the engine's (the reference's `RequestStream`,
    dynalm/src/runtime/engine.h:202-225): the engine's thread puts every event of the request into a queue of its
    own, whatever the reader does; `next` takes them out."""

    def __init__(self, engine: "Engine"):
        self._engine = engine
        self._events: "queue.Queue[Event]" = queue.Queue()
        self.request_id: Optional[int] = None
        self.finished = False

    def _put(self, ev: Event) -> None:
        self._events.put(ev)

    def next(self, timeout: Optional[float] = None) -> Optional[Event]:
        """The next event, waiting up to `timeout` seconds for it (None: for as long as it takes). None when the
        time ran out, or when the last event (`finished`) has been handed out before."""
        if self.finished:
            return None
        try:
            ev = self._events.get(timeout=timeout)
        except queue.Empty:
            return None
        if ev.finished:
            self.finished = True
        return ev

    def cancel(self) -> None:
        """Ask the engine to stop the request; its last event (status "cancelled") still arrives."""
        if self.request_id is not None and not self.finished:
            self._engine.scheduler.cancel(self.request_id)

    def __iter__(self) -> Iterator[Event]:
        while True:
            ev = self.next()
            if ev is None:
                return
            yield ev

    def tokens(self) -> List[int]:
        """Wait for the request to end; its generated tokens."""
        return [ev.token for ev in self if ev.token is not None]


class Engine:
    def __init__(self, model: Optional[str] = None, *, config: Optional[Mapping[str, Any]] = None,
                 tensors: Optional[Mapping[str, torch.Tensor]] = None, random_seed: Optional[int] = None,
                 dtype: str = "bfloat16", ctx: Optional[int] = None, batch: int = 512, max_running: int = 64,
                 page_size: int = DEFAULT_PAGE_SIZE, device: str = "cuda:0",
                 scheduler: Optional[SchedulerConfig] = None, keep_trace: bool = False):
        """model: a folder with config.json and model.safetensors. Without a folder, pass `config`
        (a config.json dict) and either `tensors` or `random_seed` (random weights in memory).
        ctx: tokens of cache over all live requests; None sizes it from the free device memory as the reference's
        kv_tokens = 0 does (dynalm/src/runtime/engine.h:63), and a size that cannot fit is refused at once with
        the largest one that would (engine/memory.py)."""
        if model is None and config is not None and tensors is None:
            if random_seed is None:
                raise InvalidArgument("a configuration without tensors needs random_seed")
            from ..registry import find_architecture
            from ..weights.random_init import random_tensors
            from .runtime import parse_dtype
            arch = find_architecture(config)
            plan = arch.plan(arch.read_config(config), present=None)
            tensors = random_tensors(plan, random_seed, parse_dtype(dtype))
        self.built: BuiltModel = build(model, config_obj=config, tensors=tensors, dtype=dtype, kv_tokens=ctx,
                                       max_batch_tokens=batch, max_requests=max_running, page_size=page_size,
                                       device=device)
        self.config = self.built.config
        self.step_fn = self.built.step_fn
        self.executor = GpuExecutor(self.step_fn)
        cfg = scheduler or SchedulerConfig()
        cfg.max_running = min(cfg.max_running, max_running)
        cfg.max_batch_tokens = min(cfg.max_batch_tokens, batch) if scheduler else batch
        cfg.context_length = min(cfg.context_length, self.built.plan.context_length)
        self.scheduler = Scheduler(self.executor, cfg, keep_trace=keep_trace)
        # the engine's own thread (see `start`): not running until asked for
        self._thread: Optional[threading.Thread] = None
        self._wake = threading.Condition()
        self._stop = False
        self.loop_error: Optional[BaseException] = None

    # ---- the engine's thread ------------------------------------------------------------------------------------
    def start(self) -> None:
        """Run the scheduler on a thread of the engine's own, as the reference's engine does
        (`Engine::loop`, dynalm/src/runtime/engine.cpp:560-627): it steps while there is work and sleeps while there
        is none; `submit` from any thread wakes it. While it runs, `generate` and `stream` hand their requests to it
        instead of stepping themselves, and nobody else may call `step`."""
        if self._thread is not None:
            return
        self._stop = False
        self.scheduler.on_submit = self._notify
        self._thread = threading.Thread(target=self._loop, name="dynalm-engine", daemon=True)
        self._thread.start()

    def _notify(self) -> None:
        with self._wake:
            self._wake.notify_all()

    def _loop(self) -> None:
        torch.cuda.set_device(self.built.runtime.device)
        while True:
            with self._wake:
                while not self._stop and self.scheduler.idle:
                    self._wake.wait()
                if self._stop:
                    return
            try:
                self.scheduler.step()
            except BaseException as e:          # nothing a request does may end the loop silently
                self.loop_error = e
                self.scheduler.cancel_all()

    def shutdown(self) -> None:
        """Cancel what is still running, let the loop deliver the last events, and stop the thread."""
        if self._thread is None:
            return
        self.scheduler.cancel_all()
        deadline = time.monotonic() + 30.0
        while not self.scheduler.idle and time.monotonic() < deadline and self._thread.is_alive():
            time.sleep(0.001)
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        self._thread.join(timeout=30.0)
        self._thread = None
        self.scheduler.on_submit = None

    def submit(self, prompt: Sequence[int], max_tokens: int = 128, sampling: Optional[SamplingParams] = None,
               stop_token_ids: Sequence[int] = (), priority: int = 0, timeout_ms: float = 0.0) -> RequestStream:
        """Hand a request to the engine's thread (started if it is not running) from any thread; the events come
        back through the returned stream (the reference's `Engine::submit` / `generate_text`,
        dynalm/src/runtime/engine.h:292-343)."""
        self.start()
        stream = RequestStream(self)
        stream.request_id = self.scheduler.submit(Request(list(prompt), max_tokens, sampling or SamplingParams(),
                                                          tuple(stop_token_ids), on_event=stream._put,
                                                          priority=priority, timeout_ms=timeout_ms))
        return stream

    # ---- generation ------------------------------------------------------------------------------------
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], max_tokens: int = 128,
                 temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                 repeat_penalty: float = 1.0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                 repeat_last_n: int = 64, seed: Optional[int] = None, stop_token_ids: Sequence[int] = (),
                 sampling: Optional[Sequence[SamplingParams]] = None) -> Union[Generation, List[Generation]]:
        """Generate for one prompt (a list of ids) or several (a list of lists), batched continuously.
        `seed` seeds request i with seed + i. `sampling` overrides the sampling options per prompt."""
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if self._thread is not None:
            return self._generate_on_loop(plist, single, max_tokens, temperature, top_k, top_p, min_p, repeat_penalty,
                                          presence_penalty, frequency_penalty, repeat_last_n, seed, stop_token_ids,
                                          sampling)
        results: Dict[int, Generation] = {}
        first: Dict[int, float] = {}
        t0 = time.perf_counter()
        order = []
        for i, p in enumerate(plist):
            sp = sampling[i] if sampling is not None else SamplingParams(
                temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=repeat_penalty,
                presence_penalty=presence_penalty, frequency_penalty=frequency_penalty, penalty_last_n=repeat_last_n,
                seed=None if seed is None else seed + i)
            order.append(self.scheduler.submit(Request(p, max_tokens, sp, tuple(stop_token_ids))))
        toks: Dict[int, List[int]] = {rid: [] for rid in order}
        while not self.scheduler.idle:
            for ev in self.scheduler.step():
                if ev.request_id not in toks:
                    continue
                if ev.token is not None:
                    toks[ev.request_id].append(ev.token)
                    first.setdefault(ev.request_id, (time.perf_counter() - t0) * 1e3)
                if ev.finished:
                    results[ev.request_id] = Generation(toks[ev.request_id], ev.finish_reason, ev.status, ev.error,
                                                        ev.prompt_tokens, first.get(ev.request_id, 0.0),
                                                        (time.perf_counter() - t0) * 1e3)
        out = [results[rid] for rid in order]
        return out[0] if single else out

    def _generate_on_loop(self, plist, single, max_tokens, temperature, top_k, top_p, min_p, repeat_penalty,
                          presence_penalty, frequency_penalty, repeat_last_n, seed, stop_token_ids, sampling):
        t0 = time.perf_counter()
        streams = []
        for i, p in enumerate(plist):
            sp = sampling[i] if sampling is not None else SamplingParams(
                temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p, repetition_penalty=repeat_penalty,
                presence_penalty=presence_penalty, frequency_penalty=frequency_penalty, penalty_last_n=repeat_last_n,
                seed=None if seed is None else seed + i)
            streams.append(self.submit(p, max_tokens, sp, stop_token_ids))
        out = []
        for s in streams:
            toks, first, last = [], 0.0, None
            for ev in s:
                if ev.token is not None:
                    toks.append(ev.token)
                    first = first or (time.perf_counter() - t0) * 1e3
                last = ev
            out.append(Generation(toks, last.finish_reason, last.status, last.error, last.prompt_tokens, first,
                                  (time.perf_counter() - t0) * 1e3))
        return out[0] if single else out

    def stream(self, prompt: Sequence[int], max_tokens: int = 128, sampling: Optional[SamplingParams] = None,
               stop_token_ids: Sequence[int] = (), priority: int = 0, timeout_ms: float = 0.0) -> Iterator[Event]:
        """Events of one request as they come (the counterpart of RequestStream::next; priority and timeout_ms
        as GenerateParams, dynalm/src/runtime/engine.h:176-225)."""
        if self._thread is not None:
            yield from self.submit(prompt, max_tokens, sampling, stop_token_ids, priority, timeout_ms)
            return
        rid = self.scheduler.submit(Request(list(prompt), max_tokens, sampling or SamplingParams(),
                                            tuple(stop_token_ids), priority=priority, timeout_ms=timeout_ms))
        done = False
        while not done and not self.scheduler.idle:
            for ev in self.scheduler.step():
                if ev.request_id == rid:
                    yield ev
                    done = done or ev.finished

    # ---- direct access -----------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """The step function itself: logits at the wanted places (see StepFunction.step)."""
        return self.step_fn.step(entries)

    def end(self, request) -> None:
        self.step_fn.end(request)

    def fork(self, parent, child) -> None:
        """A new request that goes on from where `parent` stands, sharing its cache pages (see StepFunction.fork)."""
        self.step_fn.fork(parent, child)

    def stats(self) -> dict:
        s = self.scheduler.stats
        from ..kernels import gemm, ops
        from . import launch_memo
        fn = self.step_fn
        return {"scheduler": dict(vars(s)), "free_pages": self.built.cache.free_pages,
                "pages": self.built.cache.num_pages, "cache_bytes": self.built.cache.bytes(),
                "workspace_bytes": self.built.runtime.workspace_bytes(),
                # how the steps were issued (counts since the process began, over all engines)
                "kernel_launches": ops.LAUNCHES, "library_products": gemm.LIBRARY_CALLS,
                "layers_issued_by_address": launch_memo.REPLAYED_LAYERS,
                "graphs": {"captured": fn.graph_captures, "capture_ms": round(fn.graph_capture_ms, 3),
                           "replayed_kernel_launches": fn.graph_kernel_launches}}
