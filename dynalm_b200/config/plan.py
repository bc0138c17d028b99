"""The model plan: what an architecture's configuration turns into before anything is built.

A plan is data. It lists the parts of every layer, each with its own sizes and constants, how a block
arranges them, and the order in which layers run. Nothing in it knows which architecture produced
it; the builders in `dynalm_b200.parts` turn each spec into a part by its `kind`.

A spec says what kind of part it is, how wide the stream is that it works on, which file tensors it
takes, and whatever else that kind needs as an open set of named parameters: attention's head counts
and window, a gated feed-forward's inner width, a state-space mixer's state size. A new kind brings its
own parameters; this file has no field for any of them. Parameters read as attributes
(`spec.num_heads`), and two specs are equal (and hash alike) when kind, width and parameters are; the
tensor names do not count, so that layers of equal structure compare equal.

The reference keeps the same information in one flat `ModelConfig`
(dynalm/src/model_ir/model_config.h:48-114) read by one generic `Transformer`; here it is per layer so
that layers of one model may differ.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Mapping, Optional, Tuple


def _frozen(value: Any) -> Any:
    """Lists and dicts of parameters become tuples, so that a spec can be hashed."""
    if isinstance(value, (list, tuple)):
        return tuple(_frozen(v) for v in value)
    if isinstance(value, dict):
        return tuple(sorted((k, _frozen(v)) for k, v in value.items()))
    return value


class Spec:
    """kind, width, named parameters, file tensors (local name -> name in the model file)."""

    registry = ""          # which registry of dynalm_b200.parts builds it: "mixer", "feed_forward", "norm", "position"
    __slots__ = ("kind", "width", "params", "tensors", "_key")

    def __init__(self, kind: str, width: int = 0, tensors: Optional[Mapping[str, str]] = None, **params: Any):
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "width", int(width))
        object.__setattr__(self, "params", {k: _frozen(v) for k, v in params.items()})
        object.__setattr__(self, "tensors", dict(tensors or {}))
        object.__setattr__(self, "_key", (type(self).__name__, kind, int(width), tuple(sorted(self.params.items(), key=lambda kv: kv[0]))))

    def __getattr__(self, name: str) -> Any:
        try:
            return object.__getattribute__(self, "params")[name]
        except KeyError:
            raise AttributeError(f"{type(self).__name__} of kind '{self.kind}' has no parameter '{name}'") from None

    def __setattr__(self, name: str, value: Any) -> None:
        raise AttributeError("a spec cannot be changed once made")

    def get(self, name: str, default: Any = None) -> Any:
        return self.params.get(name, default)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, Spec) and self._key == other._key

    def __hash__(self) -> int:
        return hash(self._key)

    def __repr__(self) -> str:
        inner = ", ".join(f"{k}={v!r}" for k, v in self.params.items())
        return f"{type(self).__name__}({self.kind!r}, width={self.width}{', ' + inner if inner else ''})"


class NormSpec(Spec):
    """kind "rms": y = x / sqrt(mean(x^2) + eps) * weight."""

    registry = "norm"
    __slots__ = ()

    def __init__(self, kind: str, width: int, eps: float = 1e-6, tensors: Optional[Mapping[str, str]] = None, **params: Any):
        super().__init__(kind, width, tensors, eps=float(eps), **params)


class PositionSpec(Spec):
    """Position encoding applied to queries and keys of one mixer.

    kind "rotary" (parameters head_dim, rotary_dim, theta, pos_scale, factors): pairs (i, i + rotary_dim/2) of
    each head are rotated by `pos * pos_scale * theta**(-2i/rotary_dim) / factors[i]` (factors: one per pair, None
    = all ones); kind "none": nothing.
    """

    registry = "position"
    __slots__ = ()

    def __init__(self, kind: str, head_dim: int = 0, rotary_dim: int = 0, theta: float = 10000.0, pos_scale: float = 1.0,
                 factors: Optional[Tuple[float, ...]] = None, **params: Any):
        super().__init__(kind, 0, None, head_dim=int(head_dim), rotary_dim=int(rotary_dim), theta=float(theta),
                         pos_scale=float(pos_scale), factors=None if factors is None else tuple(factors), **params)


class MixerSpec(Spec):
    """The part of a layer that lets positions see each other. kind "attention" (parameters num_heads,
    num_kv_heads, head_dim, scale: multiplies q.k before the softmax, window: 0 = all earlier keys, n = the last n
    keys, itself included, position: a PositionSpec or None): causal grouped-query attention over a paged cache."""

    registry = "mixer"
    __slots__ = ()


class FeedForwardSpec(Spec):
    """kind "gated_mlp" (parameters inner, activation): down(act(gate(x)) * up(x))."""

    registry = "feed_forward"
    __slots__ = ()


class BlockSpec:
    """How one layer arranges its parts. `parts`: name -> spec, in the order the arrangement gives them meaning
    (kind "pre_norm": mixer_norm, mixer, ffn_norm, ffn, with x += s*mixer(norm1(x)); x += s*ffn(norm2(x)),
    s = the parameter residual_scale). Keyword arguments whose values are specs are parts, the others are
    parameters of the arrangement; both read as attributes."""

    __slots__ = ("kind", "parts", "params", "_key")

    def __init__(self, kind: str, parts: Optional[Mapping[str, Spec]] = None, **more: Any):
        named = dict(parts or {})
        params = {}
        for k, v in more.items():
            if isinstance(v, Spec):
                named[k] = v
            else:
                params[k] = _frozen(v)
        object.__setattr__(self, "kind", kind)
        object.__setattr__(self, "parts", named)
        object.__setattr__(self, "params", params)
        object.__setattr__(self, "_key", (kind, tuple(named.items()), tuple(sorted(params.items(), key=lambda kv: kv[0]))))

    def __getattr__(self, name: str) -> Any:
        parts = object.__getattribute__(self, "parts")
        if name in parts:
            return parts[name]
        params = object.__getattribute__(self, "params")
        if name in params:
            return params[name]
        raise AttributeError(f"block of kind '{self.kind}' has neither a part nor a parameter '{name}'")

    def __setattr__(self, name: str, value: Any) -> None:
        raise AttributeError("a spec cannot be changed once made")

    def get(self, name: str, default: Any = None) -> Any:
        return self.params.get(name, default)

    def __iter__(self) -> Iterator[Tuple[str, Spec]]:
        return iter(self.parts.items())

    def __eq__(self, other: object) -> bool:
        return isinstance(other, BlockSpec) and self._key == other._key

    def __hash__(self) -> int:
        return hash(self._key)

    def __repr__(self) -> str:
        return f"BlockSpec({self.kind!r}, parts={list(self.parts)}, params={self.params})"


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
