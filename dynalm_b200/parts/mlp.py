"""Gated feed-forward: down(act(gate x) * up x), the "gated_mlp" kind
(dynalm/src/model/transformer.cpp:671-693). Gate and up run as one product against [Wg; Wu]."""

from __future__ import annotations

from typing import Dict

import torch

from ..errors import Unsupported
from ..kernels import ops
from ..kernels.gemm import linear_partial, linear_swiglu
from .base import TensorDecl, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts (and graph_key) only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {
            "gate": TensorDecl((spec.inner, spec.width)),
            "up": TensorDecl((spec.inner, spec.width)),
            "down": TensorDecl((spec.width, spec.inner)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if spec.get("activation", "silu") != "silu":
            raise Unsupported(f"gated_mlp: activation '{spec.get('activation')}' has no kernel (silu does)")
        self.spec = spec
        self.rt = runtime
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"]

    def first_weights(self) -> torch.Tensor:
        """The weights this part streams first (a block may say so to the kernel in front, kernels/ops.stream_ahead)."""
        return self.w_gate_up

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        s, rt = self.spec, self.rt
        if x.shape[0] <= ops.SKINNY_FAST_ROWS:
            ops.stream_ahead(self.w_down)              # taken by the gate | up product, read by the product after it
        act = linear_swiglu(x, self.w_gate_up, rt, s.inner)
        return linear_partial(act, self.w_down, rt, "ffn_out")
