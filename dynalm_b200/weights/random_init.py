"""Seeded random weights for a configuration, and a writer of whole model folders.

The reference has no such mode in the engine; its tests synthesize files
(dynalm/tests/tiny_gguf.h:254-311: matrices from a seeded generator, norm weights 1 + 0.1 u).
Here matrices are N(0, 0.02) and norm weights 1 + N(0, 0.1), drawn per tensor from a
generator keyed by (seed, tensor name), so a tensor's values do not depend on which other
tensors exist or in which order they are made.
"""

from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping

import torch

from ..config.plan import ModelPlan
from ..registry import find_architecture
from .loader import expected_tensors
from .safetensors import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensors(plan: ModelPlan, seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """CPU tensors for every tensor the plan declares. Values are drawn in float32 and then
    rounded to `dtype`, so the bfloat16 and float32 files of one seed differ only by that rounding."""
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected_tensors(plan).items():
        g = torch.Generator(device="cpu")
        g.manual_seed(_tensor_seed(seed, name))
        if decl.role == "table_int" or decl.init == "zeros":
            out[name] = torch.zeros(decl.shape, dtype=torch.int32 if decl.role == "table_int" else dtype)
            continue
        t = torch.empty(decl.shape, dtype=torch.float32)
        if decl.init == "around_one":
            t.normal_(0.0, NORM_STD, generator=g).add_(1.0)
        else:
            t.normal_(0.0, MATRIX_STD, generator=g)
        out[name] = t.to(dtype)
    return out


def write_model_folder(folder: str, config_obj: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> None:
    """Write config.json and model.safetensors for `config_obj` (a config.json dict) with
    random weights of `seed`. An untied head gets its own lm_head tensor."""
    arch = find_architecture(config_obj)
    config = arch.read_config(config_obj)
    plan = arch.plan(config, present=None)
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(plan, seed, dtype)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config_obj), f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
