"""Causal grouped-query attention over the paged cache: the "attention" mixer.

Order of work as the reference's layer body (dynalm/src/model/transformer.cpp:607-654): q, k, v
projections (here one product against the row-wise concatenation [Wq; Wk; Wv], which changes no
result), position encoding of q and k, write of k and v into the cache, attention of every row over
its request's keys, output projection. The mixer keeps sizes and constants from its spec only.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import POSITIONS, CacheSpec, TensorDecl, register_mixer


@register_mixer("attention")
class PagedAttention:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts (and graph_key) only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        qw, kw = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return {
            "q": TensorDecl((qw, spec.width)),
            "k": TensorDecl((kw, spec.width)),
            "v": TensorDecl((kw, spec.width)),
            "o": TensorDecl((spec.width, qw)),
            "q_bias": TensorDecl((qw,), role="vector", required=False, init="bias"),
            "k_bias": TensorDecl((kw,), role="vector", required=False, init="bias"),
            "v_bias": TensorDecl((kw,), role="vector", required=False, init="bias"),
            "o_bias": TensorDecl((spec.width,), role="vector", required=False, init="bias"),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if spec.head_dim % 16 or not 0 < spec.head_dim <= 256:
            raise Unsupported(f"attention: head_dim {spec.head_dim} must be a multiple of 16, at most 256")
        if spec.num_heads % spec.num_kv_heads:
            raise Unsupported(f"attention: {spec.num_heads} heads do not divide into {spec.num_kv_heads} KV heads")
        self.spec = spec
        self.rt = runtime
        self.q_width = spec.num_heads * spec.head_dim
        self.kv_width = spec.num_kv_heads * spec.head_dim
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        biases = [tensors.get("q_bias"), tensors.get("k_bias"), tensors.get("v_bias")]
        if any(b is not None for b in biases):
            widths = (self.q_width, self.kv_width, self.kv_width)
            self.b_qkv = torch.cat([b if b is not None else torch.zeros(w, dtype=torch.float32, device=runtime.device)
                                    for b, w in zip(biases, widths)]).contiguous()
        else:
            self.b_qkv = None
        self.w_o = tensors["o"]
        self.b_o = tensors.get("o_bias")
        pos = spec.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if pos is not None else None

    def step_plans(self) -> list:
        """What this mixer wants worked out once per step on the host and sent with the step's integers: the query
        tiles of its prompt kernels (kernels/attention.py)."""
        from ..kernels import attention as fast
        plans = [fast.QUERY_TILES]
        if fast.DECODE_PLANNED and fast.decode_uses_tensor_cores(self.spec):
            plans.append(fast.decode_units_plan(self.spec))
        if fast.TILE_PARTS and self.spec.head_dim in ops.PREFILL_TCGEN05_HEAD_DIMS:
            plans.append(fast.tile_parts_plan(self.spec))
        return plans

    def first_weights(self) -> torch.Tensor:
        """The weights this part streams first (a block may say so to the kernel in front, kernels/ops.stream_ahead)."""
        return self.w_qkv

    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec(kind="pages", entry_shape=(self.spec.num_kv_heads, self.spec.head_dim), tensors=2,
                         window=self.spec.get("window", 0))

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] normed input in the compute dtype -> [rows, width]."""
        s, rt = self.spec, self.rt
        rows = x.shape[0]
        k_cache, v_cache = cache.arrays
        table = self.position.table() if self.position is not None else None
        if owns_cache and self._fused_projection_applies(x, table):
            # one kernel projects, rotates and writes the cache
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))
            step_angles = getattr(self.position, "step_angles", None)
            angles = step_angles(ctx, rt) if rows > ops.SKINNY_FAST_ROWS and step_angles is not None else None
            ops.gemm_qkv_rope(x, self.w_qkv, qkv, ctx.positions, ctx.row_slot, cache.block_table, k_cache, v_cache,
                              table[0], table[2], s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, angles)
            return self._attend_and_project(qkv, cache, ctx, rows)
        if owns_cache:
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))
            linear(x, self.w_qkv, qkv, self.b_qkv)
        else:
            # a layer that reads another entry's cache makes queries only
            qkv = rt.buffer("attn_qkv", (rows, self.q_width + 2 * self.kv_width))[:, :self.q_width]
            linear(x, self.w_qkv[:self.q_width], qkv, self.b_qkv[:self.q_width] if self.b_qkv is not None else None)
        if self.position is not None and table is None:
            q = qkv[:, :self.q_width].unflatten(1, (s.num_heads, s.head_dim))
            k = qkv[:, self.q_width:self.q_width + self.kv_width].unflatten(1, (s.num_kv_heads, s.head_dim)) \
                if owns_cache else None
            self.position.apply(q, k, ctx.positions[:rows])
        inv_freq, rot, pos_scale = table if table is not None else (None, 0, 1.0)
        ops.rope_cache_write(qkv, ctx.positions, ctx.row_slot, cache.block_table, k_cache, v_cache, inv_freq, rot,
                             pos_scale, s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, write_cache=owns_cache)
        return self._attend_and_project(qkv, cache, ctx, rows)

    def _fused_projection_applies(self, x: torch.Tensor, table) -> bool:
        """bfloat16, no bias, the rotation covers the whole head, and either few rows (the weight-streaming
        kernel) or enough tiles for the tcgen05 kernel with a head size it takes (ops.QKV_ROPE_TCGEN05_MIN_ROUNDS)."""
        if not (table is not None and table[0] is not None and table[1] == self.spec.head_dim and self.b_qkv is None
                and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0):
            return False
        if x.shape[0] <= ops.SKINNY_FAST_ROWS:
            return True
        from ..kernels.gemm import rotating_epilogue_pays, tcgen05_ok
        if not rotating_epilogue_pays(x.shape[0], self.w_qkv.shape[0], self.spec.head_dim):
            return False
        qkv = self.rt.buffer("attn_qkv", (x.shape[0], self.q_width + 2 * self.kv_width))
        return tcgen05_ok(x, self.w_qkv, qkv, self.w_qkv.shape[0])

    def _attend_and_project(self, qkv: torch.Tensor, cache, ctx, rows: int) -> torch.Tensor:
        s, rt = self.spec, self.rt
        attn = rt.buffer("attn_out", (rows, self.q_width))
        if rows <= ops.SKINNY_FAST_ROWS:
            ops.stream_ahead(self.w_o)                 # taken by the decode attention, read by the product after it
        self.attend(qkv, cache, ctx, attn)
        ops.stream_ahead(None)
        if self.b_o is None:
            return linear_partial(attn, self.w_o, rt, "mixer_out")
        out = rt.buffer("mixer_out", (rows, s.width))
        linear(attn, self.w_o, out, self.b_o)
        return out

    def graph_key(self, ctx) -> tuple:
        from ..kernels import attention as fast
        if fast.DECODE_PLANNED and fast.decode_uses_tensor_cores(self.spec):
            planned = ctx.extras.get(fast.decode_units_plan(self.spec).name)
            if planned is not None and planned[1][0] > 0:
                return ()         # the grid of the planned decode kernel depends on the number of rows alone
        return (("attn_splits", fast.decode_plan(ctx, self.spec)),)

    def attend(self, qkv: torch.Tensor, cache, ctx, out: torch.Tensor) -> None:
        s = self.spec
        k_cache, v_cache = cache.arrays
        from ..kernels import attention as fast
        if fast.paged_attention(qkv, cache, ctx, out, s, self.rt):
            return
        ops.paged_attention_generic(qkv, k_cache, v_cache, cache.block_table, ctx.positions, ctx.row_slot, out,
                                    s.num_heads, s.num_kv_heads, s.head_dim, cache.page_size, float(s.scale), s.get("window", 0))
