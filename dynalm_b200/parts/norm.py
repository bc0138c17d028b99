"""RMSNorm over the float32 residual stream (CpuDevice::rms_norm, dynacore/cpu/cpu_device.cpp:1179-1205)."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from .base import TensorDecl, register_norm


@register_norm("rms")
class RMSNorm:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.width,), role="vector", init="around_one")}

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        self.spec = spec
        self.weight = tensors["weight"]
        self.eps = float(spec.eps)

    def forward(self, residual: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
                delta_scale: float = 1.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """out = norm(residual + delta_scale * delta); the sum is written back to `residual` unless
        `rows` picks a subset. Everything is computed in float32; `out` has the compute dtype."""
        ops.rmsnorm(residual, self.weight, self.eps, out, delta=delta, delta_scale=delta_scale, rows=rows)
        return out
