"""y = x W^T (+ bias): picks the matrix-product kernel for a dtype and shape.

float32 always runs the plain fixed-order kernel (csrc/gemm_simt.cu): the true 32-bit path uses no
tensor cores and no reduced-precision mode. bfloat16 with at most 16 rows (decode) runs a
weight-streaming kernel, which can also apply SwiGLU on the way out or leave split-K partial sums for
the consumer to add: the mma.sync one (csrc/gemm_skinny.cu) up to 8 rows, the tcgen05 one
(csrc/gemm_stream_tcgen05.cu), which computes the product transposed, from 9 to 16 rows. bfloat16 with
more rows runs the tcgen05 / TMEM / TMA kernel (csrc/gemm_tcgen05.cu, plain or with the SwiGLU
epilogue) whenever the product has enough 128 x 128 tiles to fill the GPU; the few shapes in between
(17..127 rows with a narrow output, where split-K wins) run the library product (cuBLAS through torch), which is where the reference's GPU path calls a library too
(ggml_mul_mat, dynacore/src/gpu/ggml_graph.cpp:278-292). Shapes none of these can express (a bias, a K
that is no multiple of 8) run the plain kernel.
"""

from __future__ import annotations

from typing import Optional

import os

import torch

from . import ops
from .device import sm_count

_mm_out_dtype_ok: Optional[bool] = None
LIBRARY_CALLS = 0    # matrix products handed to the library so far


def _mm_f32_out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """bf16 x bf16 -> fp32 through the library, when this torch offers it."""
    global _mm_out_dtype_ok
    if _mm_out_dtype_ok is False:
        return False
    ops.note_unrecorded_work()
    try:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        _mm_out_dtype_ok = True
        return True
    except (TypeError, RuntimeError):
        if _mm_out_dtype_ok is None:
            _mm_out_dtype_ok = False
            return False
        raise


def skinny_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[0] <= ops.SKINNY_FAST_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous())


# Row counts (9 .. STREAM_ROWS) that the tcgen05 streaming kernel takes. Measured inside whole decode steps on B200
# (1B shapes, 1,024 tokens of context): at 16 rows the step takes 0.98 ms with it against 1.09 ms with the mma.sync
# kernel; at 8 rows 0.91 against 0.89 ms; at 24 rows 1.11 against 1.12 ms; at 32 and 64 rows the library's split-K
# kernels are faster (1.15 against 1.18 ms, 1.41 against 1.49 ms): the consumer of the partial sums (one block per
# row) pays for them.
STREAM_ROWS = min(int(os.environ.get("DYNALM_STREAM_ROWS", "16")), ops.STREAM_MAX_ROWS)


def use_stream(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and 8 < x.shape[0] <= STREAM_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0)


STREAM_MAX_SPLITS = 6      # more partial sums cost the norm that adds them more than they save (0.98 against 1.00 ms)


def stream_split_count(n_features: int, k: int) -> int:
    """K splits of the streaming kernel so that its blocks (one per 128 features and split) about fill the GPU, every
    split with at least four 64-wide slices of K."""
    tiles = -(-n_features // 128)
    want = max(1, (sm_count() + tiles // 2) // tiles)
    return max(1, min(want, STREAM_MAX_SPLITS, k // 256))


def split_count(n_features: int, k: int, rows: int) -> int:
    """How many blocks split K for a small N, so that the grid covers the GPU about twice and every
    warp of a block still gets at least one 64-wide piece of K."""
    tiles = -(-n_features // (16 if rows <= 16 else 32))
    want = -(-2 * sm_count() // tiles)
    return max(1, min(want, 8, k // 512))


def tcgen05_ok(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, features: int) -> bool:
    """Whether the tcgen05 kernel takes this product and has enough tiles to fill the GPU: with few
    tiles (few rows and a narrow output) a split-K library kernel does better."""
    if x.dtype != torch.bfloat16 or x.shape[1] % 8 or x.stride(1) != 1 or x.stride(0) % 8 or not w.is_contiguous():
        return False
    if x.data_ptr() % 16 or w.data_ptr() % 16 or out.data_ptr() % 16 or out.stride(1) != 1:
        return False
    align = 4 if out.dtype == torch.float32 else 8
    if features % align or out.stride(0) % align:
        return False
    tiles = -(-x.shape[0] // 128) * -(-features // 128)      # at the narrowest tile the kernel may choose
    return tiles >= 96


def rotating_epilogue_pays(rows: int, features: int, head_dim: int) -> bool:
    """Whether the q | k | v product over `rows` rows should rotate and write the cache in its own epilogue (the
    tcgen05 kernel): the head size is one it takes and its tiles make enough rounds over the SMs to hide that
    epilogue (ops.QKV_ROPE_TCGEN05_MIN_ROUNDS); otherwise the product is followed by the rotation kernel."""
    if head_dim not in ops.QKV_ROPE_TCGEN05_HEAD_DIMS:
        return False
    tiles = -(-rows // 128) * -(-features // 256)
    return tiles >= ops.QKV_ROPE_TCGEN05_MIN_ROUNDS[head_dim] * sm_count()


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_scale: float = 1.0) -> torch.Tensor:
    """out[M, N] = (x[M, K] @ w[N, K].T + bias[N]) * out_scale. x and w share a dtype; out may be
    float32 for bfloat16 operands (logits)."""
    global LIBRARY_CALLS
    if x.dtype == torch.float32 or bias is not None:
        ops.gemm_simt(x, w, out, bias, out_scale)
        return out
    if use_stream(x, w) and out.stride(1) == 1:
        ops.gemm_stream(x, w, out, "store", out_scale)
        return out
    if skinny_ok(x, w) and out.stride(1) == 1:
        ops.gemm_skinny(x, w, out, "store", out_scale)
        return out
    if tcgen05_ok(x, w, out, w.shape[0]):
        ops.gemm_tcgen05(x, w, out, "store", out_scale)
        return out
    if out_scale != 1.0 or not x.is_contiguous() or not out.is_contiguous():
        ops.gemm_simt(x, w, out, bias, out_scale)
        return out
    if out.dtype == x.dtype:
        ops.library_mm(x, w, out)
        LIBRARY_CALLS += 1
        return out
    if _mm_f32_out(x, w, out):
        LIBRARY_CALLS += 1
    else:
        ops.gemm_simt(x, w, out, None, 1.0)
    return out


def linear_partial(x: torch.Tensor, w: torch.Tensor, runtime, name: str) -> torch.Tensor:
    """x W^T whose consumer adds it into the residual stream: for few rows the product may split K
    and come back as float32 partial sums [parts, M, N] (see ops.rmsnorm's `delta`); otherwise a
    plain [M, N] tensor in the compute dtype."""
    M, N = x.shape[0], w.shape[0]
    if x.dtype == torch.bfloat16 and (use_stream(x, w) or skinny_ok(x, w)):
        stream = use_stream(x, w)
        parts = stream_split_count(N, x.shape[1]) if stream else split_count(N, x.shape[1], M)
        if parts > 1:
            flat = runtime.flat(f"{name}_parts_{N}", 16 * ops.SKINNY_MAX_ROWS * N, torch.float32)
            out = flat[:parts * M * N].view(parts, M, N)
            (ops.gemm_stream if stream else ops.gemm_skinny)(x, w, out, "store", 1.0)
            return out
    out = runtime.buffer(name, (M, N))
    return linear(x, w, out)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, runtime, inner: int) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) with w_gate_up = [Wg; Wu]: fused in the product's epilogue for few
    bfloat16 rows, else the product followed by the activation kernel."""
    rows = x.shape[0]
    act = runtime.buffer("ffn_act", (rows, inner))
    if x.dtype == torch.bfloat16 and use_stream(x, w_gate_up):
        ops.gemm_stream(x, w_gate_up, act, "swiglu")
        return act
    if x.dtype == torch.bfloat16 and skinny_ok(x, w_gate_up):
        ops.gemm_skinny(x, w_gate_up, act, "swiglu")
        return act
    if x.dtype == torch.bfloat16 and inner % 8 == 0 and w_gate_up.shape[0] == 2 * inner and tcgen05_ok(x, w_gate_up, act, 2 * inner):
        ops.gemm_tcgen05(x, w_gate_up, act, "swiglu")
        return act
    gate_up = runtime.buffer("ffn_gate_up", (rows, 2 * inner))
    linear(x, w_gate_up, gate_up)
    ops.silu_mul(gate_up, act)
    return act
