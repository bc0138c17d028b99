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
from .base import FEED_FORWARDS, MIXERS, NORMS, pick_tensors, register_block


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


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, spec, store, runtime):
        self.spec = spec
        self.rt = runtime
        self.mixer_norm = NORMS.get(spec.mixer_norm.kind)(spec.mixer_norm, pick_tensors(spec.mixer_norm, store, NORMS), runtime)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, pick_tensors(spec.mixer, store, MIXERS), runtime)
        self.ffn_norm = NORMS.get(spec.ffn_norm.kind)(spec.ffn_norm, pick_tensors(spec.ffn_norm, store, NORMS), runtime)
        self.ffn = FEED_FORWARDS.get(spec.ffn.kind)(spec.ffn, pick_tensors(spec.ffn, store, FEED_FORWARDS), runtime)
        self.scale = float(spec.residual_scale)
        # whether a later layer of the same kind may re-issue this block's launches by address (engine/launch_memo.py):
        # only if every part says so of itself
        parts = [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, getattr(self.mixer, "position", None)]
        self.replay_safe = all(getattr(p, "replay_safe", False) for p in parts if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()


    def forward(self, stream: ResidualStream, ctx, cache, owns_cache: bool) -> ResidualStream:
        rows, width = stream.x.shape
        h = self.rt.buffer("normed", (rows, width))
        self.mixer_norm.forward(stream.x, h, delta=stream.pending, delta_scale=stream.pending_scale)
        a = self.mixer.forward(h, ctx, cache, owns_cache)
        h = self.rt.buffer("normed", (rows, width))
        self.ffn_norm.forward(stream.x, h, delta=a, delta_scale=self.scale)
        f = self.ffn.forward(h, ctx)
        stream.pending, stream.pending_scale = f, self.scale
        return stream
