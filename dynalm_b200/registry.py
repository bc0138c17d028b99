"""One registry from an architecture's name to what builds its model.

The reference keeps a static array of adapters looked up by id
(dynalm/src/model/architecture.cpp:112-125) and keys Hugging Face folders on `model_type`
(dynalm/src/loader/hf/hf_model.cpp:160-171). Here the key is `architectures[0]` of
config.json, with `model_type` as the fallback when that list is absent.
"""

from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Protocol, Tuple

from .config.plan import ModelPlan
from .errors import Corrupt, Unsupported


class Architecture(Protocol):
    """What a registered architecture provides.

    name          the string found in config.json `architectures`
    model_types   `model_type` values that select it when `architectures` is absent
    read_config   config.json dict -> typed configuration
    plan          typed configuration (+ names of the tensors present) -> ModelPlan
    """

    name: str
    model_types: Tuple[str, ...]

    def read_config(self, obj: Mapping[str, Any]) -> Any: ...

    def plan(self, config: Any, present: Optional[set] = None) -> ModelPlan: ...


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def find_architecture(config_obj: Mapping[str, Any]) -> Architecture:
    """Pick the architecture for a parsed config.json."""
    if not isinstance(config_obj, Mapping):
        raise Corrupt("config.json is not an object")
    names = config_obj.get("architectures")
    if isinstance(names, list) and names and isinstance(names[0], str):
        arch = _ARCHITECTURES.get(names[0])
        if arch is None:
            raise Unsupported(f"architecture '{names[0]}' is not supported; registered: "
                              f"{', '.join(registered_architectures())}")
        return arch
    model_type = config_obj.get("model_type")
    if not isinstance(model_type, str):
        raise Corrupt("config.json: missing model_type")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise Unsupported(f"Hugging Face model_type '{model_type}' is not supported; registered architectures: "
                      f"{', '.join(registered_architectures())}")
