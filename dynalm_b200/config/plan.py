"""The model plan: what an architecture's configuration turns into before anything is built.

A plan is data. It lists the parts of every layer (mixer, feed-forward, norms, position
encoding and how a block arranges them), each with its own sizes and constants, and the order
in which layers run. Nothing in it knows which architecture produced it; the builders in
`dynalm_b200.parts` turn each spec into a part by its `kind`.

The reference keeps the same information in one flat `ModelConfig`
(dynalm/src/model_ir/model_config.h:48-114) read by one generic `Transformer`; here it is
per layer so that layers of one model may differ.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    kind: str                      # "rms"
    width: int
    eps: float
    tensors: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)  # local -> file name


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys of one mixer.

    kind "rotary": pairs (i, i + rotary_dim/2) of each head are rotated by
    `pos * pos_scale * theta**(-2i/rotary_dim) / factors[i]`; kind "none": nothing.
    """

    kind: str
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    pos_scale: float = 1.0
    factors: Optional[Tuple[float, ...]] = None     # one per pair, None = all ones


@dataclass(frozen=True)
class MixerSpec:
    """kind "attention": causal grouped-query attention over a paged cache."""

    kind: str
    width: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 0.0             # multiplies q.k before softmax
    window: int = 0                # 0 = all earlier keys; n = the last n keys, itself included
    position: Optional[PositionSpec] = None
    tensors: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    """kind "gated_mlp": down(act(gate(x)) * up(x))."""

    kind: str
    width: int
    inner: int = 0
    activation: str = "silu"
    tensors: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class BlockSpec:
    """kind "pre_norm": x += s*mixer(norm1(x)); x += s*ffn(norm2(x)), s = residual_scale."""

    kind: str
    mixer_norm: NormSpec
    mixer: MixerSpec
    ffn_norm: NormSpec
    ffn: FeedForwardSpec
    residual_scale: float = 1.0


@dataclass(frozen=True)
class LayerRun:
    """One entry of the run order.

    `layer` indexes `ModelPlan.layers`; the same layer may be named by several entries.
    `cache_of` is None when the entry keeps a cache of its own, or the index of an earlier
    entry whose cache it reads instead of writing one.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab: int
    width: int
    scale: float = 1.0
    tensors: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class HeadSpec:
    """Final projection to the vocabulary. `tied` uses the embedding table; logits are
    divided by `logit_divisor` (dynalm/src/model/transformer.cpp:719)."""

    vocab: int
    width: int
    tied: bool
    logit_divisor: float = 1.0
    tensors: Dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass
class ModelPlan:
    embedding: EmbeddingSpec
    layers: List[BlockSpec]
    order: List[LayerRun]
    final_norm: NormSpec
    head: HeadSpec
    context_length: int
    # File tensors that may be present but are not used (none for Llama).
    ignorable: Tuple[str, ...] = ()

    def validate(self) -> None:
        from ..errors import InvalidArgument
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise InvalidArgument(f"run order entry {i} names layer {run.layer}, the plan has {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise InvalidArgument(f"run order entry {i} reads the cache of entry {run.cache_of}, which is not earlier")
                if self.order[run.cache_of].cache_of is not None:
                    raise InvalidArgument(f"run order entry {i} reads the cache of entry {run.cache_of}, which owns none")
