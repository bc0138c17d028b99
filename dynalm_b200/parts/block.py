"""How a layer arranges its parts around the residual stream.

"pre_norm" (Llama): x += s * mixer(norm1(x)); x += s * ffn(norm2(x)), s the residual scale
(dynalm/src/model/transformer.cpp:602-697). The residual stream is float32; the sum of a part's
output into it is fused into the norm that follows, so a block leaves its last output pending.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import ops
from .base import build_part, register_block


@dataclass
class ResidualStream:
    """x: float32 [rows, width]. `pending` (compute dtype) times `pending_scale` is still to be added."""

    x: torch.Tensor
    pending: Optional[torch.Tensor] = None
    pending_scale: float = 1.0

    def flush(self) -> torch.Tensor:
        if self.pending is not None:
            ops.residual_add(self.x, self.pending, self.pending_scale)
            self.pending = None
        return self.x


class Block:
    """What every arrangement shares: it builds the parts its spec lists (each from the registry its spec names,
    kept as attributes under the spec's names), and answers for them where the engine asks a layer as a whole:
    which cache it keeps, whether its launches may be captured in a CUDA graph or re-issued by address."""

    cache_part = "mixer"        # the name of the part whose cache_spec() is the layer's

    def __init__(self, spec, store, runtime):
        self.spec = spec
        self.rt = runtime
        self.part_names = list(spec.parts)
        for name, part_spec in spec.parts.items():
            setattr(self, name, build_part(part_spec, store, runtime))
        parts = self.parts()
        # only if every part says so of itself (a position encoding that a mixer holds included)
        inner = [getattr(p, "position", None) for p in parts]
        self.replay_safe = all(getattr(p, "replay_safe", False) for p in parts + [p for p in inner if p is not None])
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts)

    def parts(self):
        return [getattr(self, n) for n in self.part_names]

    def cache_spec(self):
        part = getattr(self, self.cache_part, None)
        return part.cache_spec() if part is not None and hasattr(part, "cache_spec") else None

    def step_plans(self) -> list:
        return [plan for p in self.parts() for plan in (p.step_plans() if hasattr(p, "step_plans") else [])]

    def graph_key(self, ctx) -> tuple:
        key = ()
        for p in self.parts():
            f = getattr(p, "graph_key", None)
            if f is not None:
                key += tuple(f(ctx))
        return key


@register_block("pre_norm")
class PreNormBlock(Block):
    """parts: mixer_norm, mixer, ffn_norm, ffn; parameter: residual_scale (default 1)."""

    def __init__(self, spec, store, runtime):
        super().__init__(spec, store, runtime)
        self.scale = float(spec.get("residual_scale", 1.0))

    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        few = rows <= ops.SKINNY_FAST_ROWS         # a step bound by the stream of weights: say early what comes next
        h = self.rt.buffer("normed", (rows, width))
        if few:
            ops.stream_ahead(getattr(self.mixer, "first_weights", lambda: None)())
        self.mixer_norm.forward(stream.x, h, delta=stream.pending, delta_scale=stream.pending_scale)
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        h = self.rt.buffer("normed", (rows, width))
        if few:
            ops.stream_ahead(getattr(self.ffn, "first_weights", lambda: None)())
        self.ffn_norm.forward(stream.x, h, delta=a, delta_scale=self.scale)
        f = self.ffn.forward(h, ctx)
        stream.pending, stream.pending_scale = f, self.scale
        return stream
