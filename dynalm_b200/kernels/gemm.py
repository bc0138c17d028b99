"""y = x W^T (+ bias): picks the matrix-product kernel for a dtype and shape.

float32 always runs the plain fixed-order kernel (csrc/gemm_simt.cu): the true 32-bit path uses no
tensor cores and no reduced-precision mode. bfloat16 runs the library product (cuBLAS through torch),
which is where the reference's GPU path calls a library too (ggml_mul_mat,
dynacore/src/gpu/ggml_graph.cpp:278-292), with fp32 accumulation; shapes the library call cannot
express (a bias, a float32 output from bfloat16 operands on an older torch) run the plain kernel.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops

_mm_out_dtype_ok: Optional[bool] = None
LIBRARY_CALLS = 0    # matrix products handed to the library so far


def _mm_f32_out(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """bf16 x bf16 -> fp32 through the library, when this torch offers it."""
    global _mm_out_dtype_ok
    if _mm_out_dtype_ok is False:
        return False
    try:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
        _mm_out_dtype_ok = True
        return True
    except (TypeError, RuntimeError):
        if _mm_out_dtype_ok is None:
            _mm_out_dtype_ok = False
            return False
        raise


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_scale: float = 1.0) -> torch.Tensor:
    """out[M, N] = (x[M, K] @ w[N, K].T + bias[N]) * out_scale. x and w share a dtype; out may be
    float32 for bfloat16 operands (logits)."""
    if x.dtype == torch.float32 or bias is not None or out_scale != 1.0 or not x.is_contiguous() \
            or not out.is_contiguous():
        ops.gemm_simt(x, w, out, bias, out_scale)
        return out
    global LIBRARY_CALLS
    if out.dtype == x.dtype:
        torch.mm(x, w.t(), out=out)
        LIBRARY_CALLS += 1
        return out
    if _mm_f32_out(x, w, out):
        LIBRARY_CALLS += 1
    else:
        ops.gemm_simt(x, w, out, None, 1.0)
    return out
