"""The model built from a plan: embedding, blocks run in the plan's order, final norm, head.

This is the one generic decoder the registry's architectures build (the counterpart of the
reference's `Transformer`, dynalm/src/model/transformer.h:51-179). It resolves weights once and
allocates its scratch through the runtime's workspace; `forward` looks nothing up.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.plan import ModelPlan
from ..parts import BLOCKS, NORMS
from ..parts.base import CacheSpec, pick_tensors
from ..parts.block import ResidualStream
from ..parts.embedding import LogitsHead, TokenEmbedding
from ..kernels import ops
from . import launch_memo


class Decoder:
    def __init__(self, plan: ModelPlan, store: Dict[str, torch.Tensor], runtime):
        plan.validate()
        self.plan = plan
        self.rt = runtime
        self.embedding = TokenEmbedding(plan.embedding, store, runtime)
        self.blocks = [BLOCKS.get(b.kind)(b, store, runtime) for b in plan.layers]
        self.order = list(plan.order)
        self.final_norm = NORMS.get(plan.final_norm.kind)(plan.final_norm, pick_tensors(plan.final_norm, store, NORMS),
                                                          runtime)
        self.head = LogitsHead(plan.head, store, runtime, self.embedding)
        self.vocab = plan.head.vocab
        self.width = plan.embedding.width
        # for launch_memo: blocks of equal class and spec share a number; the layouts of their tensors are filled on use
        seen: Dict[tuple, int] = {}
        self._run_kinds = [seen.setdefault((type(self.blocks[run.layer]), self.blocks[run.layer].spec), len(seen))
                           for run in self.order]
        self._run_layouts: Dict[int, tuple] = {}

    def forget_layouts(self) -> None:
        """To be called when a part has been given another tensor object after the model has run a step: the
        addresses that engine/launch_memo.py remembers for every layer are read again."""
        self._run_layouts.clear()

    @property
    def graph_safe(self) -> bool:
        """True when every mixer and feed-forward says its launches depend only on what
        `graph_key` covers, so that a decode step can be captured once and replayed."""
        return all(getattr(b, "graph_safe", False) for b in self.blocks)

    def graph_key(self, ctx) -> tuple:
        """What, beyond the numbers of rows, the parts' launch shapes depend on for this step."""
        key = ()
        for b in self.blocks:
            f = getattr(b, "graph_key", None)
            if f is not None:
                key += tuple(f(ctx))
        return tuple(sorted(set(key)))

    def step_plans(self) -> list:
        """The step plans the layers' parts ask for, each once (by name): what a part wants computed on the host once
        per step and sent along with the step's integers (engine/step.py)."""
        plans, names = [], set()
        for b in self.blocks:
            for plan in (b.step_plans() if hasattr(b, "step_plans") else []):
                if plan.name not in names:
                    names.add(plan.name)
                    plans.append(plan)
        return plans

    def cache_specs(self) -> List[Optional[CacheSpec]]:
        """Per run-order entry: the cache it owns, or None when it owns none."""
        return [None if run.cache_of is not None else self.blocks[run.layer].cache_spec() for run in self.order]

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for obj in [self.embedding, self.head, self.final_norm] + [p for b in self.blocks for p in vars(b).values()]:
            for v in vars(obj).values() if hasattr(obj, "__dict__") else ():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    n += v.numel() * v.element_size()
        return n

    def hidden(self, ctx, caches) -> ResidualStream:
        """Run embedding and all blocks; `caches[i]` is the CacheView of run-order entry i (or None)."""
        x = self.embedding.forward(ctx.token_ids, ctx.num_tokens)
        stream = ResidualStream(x)
        memo = launch_memo.LayerLaunchMemo(self._run_layouts, self._run_kinds) if launch_memo.ENABLED else None
        for i, run in enumerate(self.order):
            owner = i if run.cache_of is None else run.cache_of
            block = self.blocks[run.layer]
            if memo is None:
                stream = block.forward(stream, ctx, caches[owner], run.cache_of is None)
            else:
                stream = memo.run(i, block, stream, ctx, caches[owner], run.cache_of is None)
        return stream

    def logits(self, stream: ResidualStream, ctx, out: torch.Tensor) -> torch.Tensor:
        """Final norm and head on the wanted rows only (dynalm/src/model/transformer.cpp:701-718)."""
        n = ctx.num_logit_rows
        normed = self.rt.buffer("final_normed", (n, self.width))
        self.final_norm.forward(stream.x, normed, delta=stream.pending, delta_scale=stream.pending_scale,
                                rows=ctx.logit_rows)
        return self.head.forward(normed, out[:n])

    def choose(self, stream: ResidualStream, ctx, ids: torch.Tensor, status_to=None) -> bool:
        """The most likely token of every wanted row into `ids`, the logits never leaving the product's kernel; False
        (and nothing done) when the head cannot do that for this step."""
        n = ctx.num_logit_rows
        if n > 8 or self.rt.dtype != torch.bfloat16:
            return False
        normed = self.rt.buffer("final_normed", (n, self.width))
        if not ops.gemm_argmax_applies(normed, self.head.weight):
            return False
        self.final_norm.forward(stream.x, normed, delta=stream.pending, delta_scale=stream.pending_scale,
                                rows=ctx.logit_rows)
        return self.head.choose(normed, ids, status_to)

    def forward(self, ctx, caches, out: Optional[torch.Tensor], choose=None) -> Optional[torch.Tensor]:
        """`choose` = (ids, status_to): only the most likely token of each wanted row is wanted, on the device; the
        head then leaves the logits out when it can (None is returned), else they are returned as always."""
        stream = self.hidden(ctx, caches)
        if ctx.num_logit_rows == 0 or (out is None and choose is None):
            return None
        if choose is not None and self.choose(stream, ctx, choose[0], choose[1]):
            return None
        return self.logits(stream, ctx, out)
