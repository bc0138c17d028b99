"""Interfaces and registries of the parts a layer is put together from.

A part is built from its spec (sizes and constants, `dynalm_b200.config.plan`), the tensors
it declared, and the runtime (device, compute dtype, workspace). No part knows which model
it belongs to. A new kind is added by writing a class with the methods below and
registering it under its `kind` string; the model builder finds it through the registry.

    Mixer          declare(spec), cache_spec(), forward(x, ctx, cache, owns_cache) -> y
    FeedForward    declare(spec), forward(x, ctx) -> y
    Norm           declare(spec), forward(residual, out, delta=..., rows=...)
    Position       (built by the mixer that uses it) table() / apply(q, k, positions)
    Block          arrangement of the four above around the residual stream

The reference has one fixed arrangement inside `Transformer::forward_batch`
(dynalm/src/model/transformer.cpp:582-697) switched by flags of `ModelConfig`; the registries
here replace those flags.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import InvalidArgument, Unsupported


@dataclass(frozen=True)
class TensorDecl:
    """A tensor a part wants from the model file.

    role "matrix": kept in the compute dtype (bfloat16, or float32 on the 32-bit path);
    role "vector": small, kept as float32 whatever the file stores (the reference converts
    norm weights and biases to fp32 copies, dynalm/src/model/transformer.cpp:92-101);
    role "table_int": integer table, kept as int32.
    `init` tells the random-weights mode how to draw it: "normal" is N(0, 0.02),
    "around_one" is 1 + N(0, 0.1) (norm weights), "bias" is N(0, 0.1), "zeros" is all zero.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    required: bool = True
    init: str = "normal"


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs the cache manager to keep for it, per run-order entry.

    kind "pages": `tensors` arrays of shape [pages, page_size, *entry_shape], addressed
    through a per-request block table; `window` > 0 says that only the last `window` tokens
    are ever read, so pages wholly behind the window are given back.
    kind "state": one array [slots, *state_shape] indexed by the request's state slot,
    zeroed when a slot is handed out.
    """

    kind: str
    entry_shape: Tuple[int, ...] = ()
    tensors: int = 2
    window: int = 0
    state_shape: Tuple[int, ...] = ()
    dtype: Optional[str] = None      # None = the compute dtype; else "float32" / "bfloat16"

    def group_key(self) -> tuple:
        return (self.kind, self.entry_shape, self.tensors, self.window, self.state_shape, self.dtype)


class _Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Any] = {}

    def register(self, kind: str, cls: Any = None):
        def put(c):
            self._kinds[kind] = c
            return c
        return put(cls) if cls is not None else put

    def get(self, kind: str):
        try:
            return self._kinds[kind]
        except KeyError:
            raise Unsupported(f"no {self.what} of kind '{kind}' is registered "
                              f"(registered: {', '.join(sorted(self._kinds)) or 'none'})") from None

    def kinds(self):
        return tuple(sorted(self._kinds))


MIXERS = _Registry("mixer")
FEED_FORWARDS = _Registry("feed-forward")
NORMS = _Registry("norm")
POSITIONS = _Registry("position encoding")
BLOCKS = _Registry("block arrangement")

REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITIONS}

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position = POSITIONS.register
register_block = BLOCKS.register


def registry_of(spec) -> _Registry:
    """The registry that builds a spec, by the spec's own `registry` word."""
    try:
        return REGISTRIES[spec.registry]
    except KeyError:
        raise Unsupported(f"a spec of kind '{spec.kind}' names no registry of parts ('{spec.registry}')") from None


def build_part(spec, store: Dict[str, Any], runtime):
    """The part of a spec: its class from the registry, the tensors it declared from the store."""
    registry = registry_of(spec)
    return registry.get(spec.kind)(spec, pick_tensors(spec, store, registry), runtime)


def declared_tensors(registry: Optional[_Registry], spec) -> Dict[str, TensorDecl]:
    """File name -> declaration for one spec, using the names the plan gave it (`registry` None: the spec's own)."""
    registry = registry or registry_of(spec)
    cls = registry.get(spec.kind)
    out: Dict[str, TensorDecl] = {}
    names = getattr(spec, "tensors", {}) or {}
    for local, decl in cls.declare(spec).items():
        name = names.get(local)
        if name is None:
            if decl.required:
                raise InvalidArgument(f"{registry.what} '{spec.kind}' needs tensor '{local}' but the plan names none")
            continue
        out[name] = decl
    return out


def pick_tensors(spec, store: Dict[str, Any], registry: _Registry) -> Dict[str, Any]:
    """local name -> loaded tensor for one spec (optional tensors absent from the plan are left out)."""
    cls = registry.get(spec.kind)
    names = getattr(spec, "tensors", {}) or {}
    return {local: store[names[local]] for local in cls.declare(spec) if local in names}
