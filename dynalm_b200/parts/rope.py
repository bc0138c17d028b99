"""Position encodings a mixer can apply to its queries and keys.

"rotary": half-split rotary embedding with optional per-pair frequency divisors (llama3 scaling) and a
position scale (linear scaling), as CpuDevice::rope (dynacore/cpu/cpu_device.cpp:1228-1262). The
frequencies are made here in 32-bit floats exactly as the reference makes them,
`pow(base, -2 i / rot) / factor_i`; the rotation itself happens inside the fused kernel
(csrc/rope_cache.cu), which asks this part for `table()`.
"none": no position encoding.

A further kind implements `table()` returning None and `apply(q, k, positions)` rotating its views in
place; the attention mixer then calls `apply` before its cache write.
"""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..errors import Unsupported
from .base import register_position


@register_position("rotary")
class RotaryEncoding:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)

    def __init__(self, spec, runtime):
        if spec.rotary_dim <= 0 or spec.rotary_dim > spec.head_dim or spec.rotary_dim % 2:
            raise Unsupported(f"rotary_dim {spec.rotary_dim} invalid for head_dim {spec.head_dim}")
        half = spec.rotary_dim // 2
        base = np.float32(spec.theta)
        i = np.arange(half, dtype=np.float32)
        inv = np.power(base, (np.float32(-2.0) * i) / np.float32(spec.rotary_dim), dtype=np.float32)
        if spec.factors is not None:
            if len(spec.factors) != half:
                raise Unsupported(f"rotary encoding has {len(spec.factors)} factors for {half} pairs")
            inv = (inv / np.asarray(spec.factors, dtype=np.float32)).astype(np.float32)
        self.spec = spec
        self.inv_freq = torch.from_numpy(inv).to(runtime.device)
        self.rotary_dim = spec.rotary_dim
        self.pos_scale = float(np.float32(spec.pos_scale))

    def table(self) -> Optional[Tuple[torch.Tensor, int, float]]:
        """(inverse frequencies float32 [rotary_dim / 2], rotary_dim, position scale) for the fused kernel."""
        return self.inv_freq, self.rotary_dim, self.pos_scale

    def step_angles(self, ctx, runtime) -> torch.Tensor:
        """(cos, sin) of every pair for every row of the step, float32 [rows, rotary_dim / 2, 2]: computed once per
        step and shared by all layers with the same encoding."""
        key = ("rope_angles", self.rotary_dim, self.pos_scale, float(self.spec.theta), self.spec.factors)
        got = ctx.extras.get(key)
        if got is None:
            from ..kernels import ops
            half = self.rotary_dim // 2
            flat = runtime.flat(f"rope_angles_{abs(hash(key)) % (1 << 32):08x}", runtime.max_tokens * half * 2)
            got = flat[:ctx.num_tokens * half * 2].view(ctx.num_tokens, half, 2)
            ops.rope_angles(ctx.positions, self.inv_freq, self.pos_scale, ctx.num_tokens, got)
            ctx.extras[key] = got
        return got


@register_position("none")
class NoPosition:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)

    def __init__(self, spec, runtime):
        self.spec = spec

    def table(self):
        return None

    def apply(self, q, k, positions) -> None:
        return None
