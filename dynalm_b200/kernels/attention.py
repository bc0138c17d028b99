"""Chooses the attention kernel for a step. Returns False when only the plain kernel applies
(float32, or a shape the tensor-core kernels refuse), and the caller runs that one."""

from __future__ import annotations

import torch


def paged_attention(qkv: torch.Tensor, cache, ctx, out: torch.Tensor, spec) -> bool:
    return False
