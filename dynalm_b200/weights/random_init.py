"""Seeded random weights for a configuration, and a writer of whole model folders.

The reference has no such mode in the engine; its tests synthesize files
(dynalm/tests/tiny_gguf.h:254-311: matrices from a seeded generator, norm weights 1 + 0.1 u).
Here matrices are N(0, 0.02), norm weights 1 + N(0, 0.1) and biases N(0, 0.1), from a counter-based
generator of this file's own: element e of tensor `name` under `seed` is a pure function of
(seed, name, e), made of 64-bit integer mixing and a Box-Muller transform in double precision. So a
tensor's values depend neither on which other tensors exist, nor on the order they are made in, nor
on the random generator of any library or its version.
"""

from __future__ import annotations

import hashlib
import json
import os
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, Iterable, Mapping, Optional

import numpy as np
import torch

from ..config.plan import ModelPlan
from ..registry import find_architecture
from .loader import expected_tensors
from .safetensors import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1
BIAS_STD = 0.1

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_CHUNK = 1 << 17          # pairs per piece of work: long enough for the threads to run side by side
_TRIG_BITS = 12
_trig_tables = None


def _tensor_key(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little")


def _trig():
    """cos and sin of 2 pi k / 2^24 are put together from two tables of 4,096 angles each (the upper and the lower
    twelve bits of k) by the addition theorems: a few multiplications per value instead of a library call."""
    global _trig_tables
    if _trig_tables is None:
        k = np.arange(1 << _TRIG_BITS, dtype=np.float64)
        coarse = k * (2.0 * np.pi / (1 << _TRIG_BITS))
        fine = k * (2.0 * np.pi / (1 << (2 * _TRIG_BITS)))
        _trig_tables = (np.cos(coarse), np.sin(coarse), np.cos(fine), np.sin(fine))
    return _trig_tables


def _normal_pairs(key: int, first: int, count: int):
    """Standard normal pairs number first .. first + count - 1 of the stream `key`: the counter goes through the
    splitmix64 finalizer; its upper 24 bits give the radius and the next 24 bits the angle of a Box-Muller
    transform in double precision."""
    with np.errstate(over="ignore"):
        z = np.arange(first, first + count, dtype=np.uint64)
        z *= _GOLDEN
        z += np.uint64(key)
        z ^= z >> np.uint64(30)
        z *= _M1
        z ^= z >> np.uint64(27)
        z *= _M2
        z ^= z >> np.uint64(31)
    u1 = ((z >> np.uint64(40)).astype(np.float64) + 1.0) * (1.0 / (1 << 24))          # (0, 1]
    r = np.sqrt(-2.0 * np.log(u1))
    hi = ((z >> np.uint64(28)) & np.uint64(0xFFF)).astype(np.intp)
    lo = ((z >> np.uint64(16)) & np.uint64(0xFFF)).astype(np.intp)
    cos_c, sin_c, cos_f, sin_f = _trig()
    ca, sa, cb, sb = cos_c[hi], sin_c[hi], cos_f[lo], sin_f[lo]
    return r * (ca * cb - sa * sb), r * (sa * cb + ca * sb)


def seeded_normal(seed: int, name: str, numel: int, mean: float, std: float) -> torch.Tensor:
    """float32 [numel]: element e is mean + std * n(e), n(e) being the cosine branch (e even) or the sine branch
    (e odd) of pair e // 2."""
    out = np.empty(numel, dtype=np.float32)
    pairs = (numel + 1) // 2
    key = _tensor_key(seed, name)
    _trig()

    def piece(first: int) -> None:
        n = min(_CHUNK, pairs - first)
        a, b = _normal_pairs(key, first, n)
        part = out[2 * first:2 * (first + n)]
        part[0::2] = a * std + mean
        part[1::2] = (b * std + mean)[:part.size // 2]

    starts = range(0, pairs, _CHUNK)
    if len(starts) > 1:
        with ThreadPoolExecutor(max_workers=min(len(starts), os.cpu_count() or 1)) as pool:
            list(pool.map(piece, starts))
    else:
        for s in starts:
            piece(s)
    return torch.from_numpy(out)


def random_tensors(plan: ModelPlan, seed: int, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """CPU tensors for every tensor the plan declares (optional ones only when the plan names them). Values are
    drawn in float32 and then rounded to `dtype`, so the bfloat16 and float32 files of one seed differ only by
    that rounding."""
    out: Dict[str, torch.Tensor] = {}
    for name, decl in expected_tensors(plan).items():
        if decl.role == "table_int" or decl.init == "zeros":
            out[name] = torch.zeros(decl.shape, dtype=torch.int32 if decl.role == "table_int" else dtype)
            continue
        numel = 1
        for s in decl.shape:
            numel *= int(s)
        if decl.init == "around_one":
            t = seeded_normal(seed, name, numel, 1.0, NORM_STD)
        elif decl.init == "bias":
            t = seeded_normal(seed, name, numel, 0.0, BIAS_STD)
        else:
            t = seeded_normal(seed, name, numel, 0.0, MATRIX_STD)
        out[name] = t.view(decl.shape).to(dtype)
    return out


def write_model_folder(folder: str, config_obj: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16, optional: Optional[Iterable[str]] = None) -> None:
    """Write config.json and model.safetensors for `config_obj` (a config.json dict) with random weights of
    `seed`. An untied head gets its own lm_head tensor. `optional`: file names of tensors that the architecture
    takes when they are present (attention biases, say) and that this folder is to carry; names that the
    architecture does not know are refused."""
    arch = find_architecture(config_obj)
    config = arch.read_config(config_obj)
    wanted = set(optional or ())
    plan = arch.plan(config, present=None)
    if wanted:
        # the head and every required tensor are decided by the configuration; the optional ones by presence
        base = set(expected_tensors(plan))
        plan = arch.plan(config, present=base | wanted)
        unknown = wanted - set(expected_tensors(plan))
        if unknown:
            from ..errors import InvalidArgument
            raise InvalidArgument(f"{arch.name} takes no tensors named {', '.join(sorted(unknown))}")
    os.makedirs(folder, exist_ok=True)
    tensors = random_tensors(plan, seed, dtype)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(config_obj), f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
