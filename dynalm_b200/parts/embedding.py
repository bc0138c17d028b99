"""The two ends of the model: token embedding and the projection to logits."""

from __future__ import annotations

from typing import Dict

import torch

from ..kernels import linear, ops
from .base import TensorDecl


def declare_embedding(spec) -> Dict[str, TensorDecl]:
    return {spec.tensors["weight"]: TensorDecl((spec.vocab, spec.width))}


def declare_head(spec) -> Dict[str, TensorDecl]:
    return {} if spec.tied else {spec.tensors["weight"]: TensorDecl((spec.vocab, spec.width))}


class TokenEmbedding:
    """x[i, :] = table[token_i, :] * scale into the float32 residual stream
    (dynalm/src/model/transformer.cpp:576-577)."""

    def __init__(self, spec, store, runtime):
        self.spec = spec
        self.rt = runtime
        self.table = store[spec.tensors["weight"]]
        self.scale = float(spec.scale)

    def forward(self, token_ids: torch.Tensor, rows: int) -> torch.Tensor:
        x = self.rt.buffer("residual", (rows, self.spec.width), torch.float32)
        ops.embed(self.table, token_ids, x, self.scale)
        return x


class LogitsHead:
    """logits = normed rows x head^T / divisor, float32 [rows, vocab]
    (dynalm/src/model/transformer.cpp:703-719). `tied` uses the embedding table."""

    def __init__(self, spec, store, runtime, embedding: TokenEmbedding):
        self.spec = spec
        self.rt = runtime
        self.weight = embedding.table if spec.tied else store[spec.tensors["weight"]]
        self.out_scale = 1.0 / float(spec.logit_divisor) if spec.logit_divisor != 1.0 else 1.0

    def forward(self, normed_rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        linear(normed_rows, self.weight, out, None, self.out_scale)
        return out

    def choose(self, normed_rows: torch.Tensor, ids: torch.Tensor, status_to=None) -> bool:
        """ids[r] = the most likely token of row r (the lowest id among equals) without the logits being written, when
        the product's kernel can do that in its epilogue; False when it cannot (the caller then takes the logits)."""
        if not ops.gemm_argmax_applies(normed_rows, self.weight) or self.out_scale <= 0:
            return False
        rows = normed_rows.shape[0]
        scratch = self.rt.flat("head_argmax_parts", 2 * 8 * -(-self.spec.vocab // 16))
        ops.gemm_argmax(normed_rows, self.weight, ids, scratch, self.out_scale, status_to)
        return True
