"""Model folders: config.json + model.safetensors (or shards) -> a plan and its tensors.

Follows the reference's folder handling (`hf::locate`, dynalm/src/loader/hf/hf_model.cpp:105-142;
`load_safetensors`, dynalm/src/loader/model_loader.cpp:219-314) and its shape validation
(`validate_standard_decoder`, dynalm/src/model/architecture.cpp:30-106), except that every
problem with the tensors is collected into ONE error instead of stopping at the first.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Tuple

import torch

from ..config.plan import ModelPlan
from ..config.reader import read_json_file
from ..errors import Corrupt, EngineError, NotFound
from ..parts.base import BLOCKS, NORMS, TensorDecl, declared_tensors
from ..registry import Architecture, find_architecture
from .safetensors import SafeTensorsFile


class WeightMismatch(EngineError):
    """The tensors of a model folder do not fit its configuration.

    `missing`: names the plan needs and the file lacks; `unexpected`: names in the file
    that no part asked for; `wrong_shape`: (name, found, expected).
    """

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]]):
        self.where = where
        self.missing = missing
        self.unexpected = unexpected
        self.wrong_shape = wrong_shape
        lines = [f"{where}: tensors do not match config.json"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + "; ".join(
                f"{n} has {list(f)}, expected {list(e)}" for n, f, e in wrong_shape))
        super().__init__("\n".join(lines))


def expected_tensors(plan: ModelPlan) -> Dict[str, TensorDecl]:
    """Every file tensor the plan's parts declare, by file name."""
    from ..parts import embedding as _emb  # registers nothing; declares its own tensors

    out: Dict[str, TensorDecl] = {}
    out.update(_emb.declare_embedding(plan.embedding))
    out.update(_emb.declare_head(plan.head))
    out.update(declared_tensors(NORMS, plan.final_norm))
    for block in plan.layers:
        BLOCKS.get(block.kind)  # fails early on an unknown arrangement
        for _, part in block:
            out.update(declared_tensors(None, part))
    return out


def check_tensors(where: str, plan: ModelPlan, found: Mapping[str, Tuple[int, ...]]) -> Dict[str, TensorDecl]:
    """Compare the shapes found in a file with what the plan declares; raise one WeightMismatch."""
    want = expected_tensors(plan)
    missing = [n for n, d in want.items() if d.required and n not in found]
    unexpected = [n for n in found if n not in want and n not in plan.ignorable]
    wrong = [(n, tuple(found[n]), tuple(d.shape)) for n, d in want.items()
             if n in found and tuple(found[n]) != tuple(d.shape)]
    if missing or unexpected or wrong:
        raise WeightMismatch(where, missing, unexpected, wrong)
    return want


@dataclass
class ModelFolder:
    """A model folder opened but not yet placed on a device."""

    path: str
    config_obj: dict
    architecture: Architecture
    config: Any
    plan: ModelPlan
    files: List[SafeTensorsFile] = field(default_factory=list)
    where: Dict[str, SafeTensorsFile] = field(default_factory=dict)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def _locate_shards(folder: str) -> List[str]:
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        obj = read_json_file(index)
        wm = obj.get("weight_map")
        if not isinstance(wm, dict) or not wm:
            raise Corrupt(f"{index}: missing weight_map")
        shards = []
        for shard in wm.values():
            # shard names that leave the folder are refused (hf_model.cpp:105-142)
            if not isinstance(shard, str) or os.path.isabs(shard) or ".." in shard.split("/"):
                raise Corrupt(f"{index}: shard name {shard!r} is not a plain file name")
            p = os.path.join(folder, shard)
            if p not in shards:
                shards.append(p)
        return shards
    raise NotFound(f"{folder}: no model.safetensors and no model.safetensors.index.json")


def open_model_folder(path: str) -> ModelFolder:
    """Read config.json, pick the architecture, open the tensors and check names and shapes."""
    if not os.path.isdir(path):
        raise NotFound(f"{path}: not a folder")
    config_obj = read_json_file(os.path.join(path, "config.json"))
    arch = find_architecture(config_obj)
    config = arch.read_config(config_obj)
    files = [SafeTensorsFile(p) for p in _locate_shards(path)]
    where: Dict[str, SafeTensorsFile] = {}
    for f in files:
        for name in f.names():
            if name in where:
                raise Corrupt(f"{f.path}: tensor '{name}' is also in {where[name].path}")
            where[name] = f
    plan = arch.plan(config, present=set(where))
    found = {name: f.entries[name].shape for name, f in where.items()}
    check_tensors(path, plan, found)
    return ModelFolder(path, config_obj, arch, config, plan, files, where)


def place_tensors(plan: ModelPlan, source: Mapping[str, torch.Tensor] | ModelFolder, device: torch.device,
                  compute_dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """Copy the declared tensors to `device`: matrices in the compute dtype, vectors in float32,
    integer tables as int32. With bfloat16 as the compute dtype, a matrix stored in 16 bits is
    used as stored; on the 32-bit path everything is widened exactly."""
    want = expected_tensors(plan)
    get = source.tensor if isinstance(source, ModelFolder) else source.__getitem__
    if not isinstance(source, ModelFolder):
        check_tensors("tensors", plan, {n: tuple(t.shape) for n, t in source.items()})
    out: Dict[str, torch.Tensor] = {}
    for name, decl in want.items():
        if isinstance(source, ModelFolder):
            if name not in source.where:
                continue
        elif name not in source:
            continue
        t = get(name)
        if decl.role == "table_int":
            dtype = torch.int32
        elif decl.role == "vector":
            dtype = torch.float32
        else:
            dtype = compute_dtype
        out[name] = t.to(device=device, dtype=dtype, non_blocking=False).contiguous()
    return out
