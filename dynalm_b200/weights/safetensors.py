"""A safetensors reader and writer.

File layout: u64 little-endian header length, a JSON header (`name -> {dtype, shape,
data_offsets}` plus an optional `__metadata__`), then the data. The reader maps the file and
refuses headers that cannot be right, with the checks of the reference's reader
(dynalm/src/loader/safetensors/safetensors.cpp:13,47-128): header length at most 100 MiB and
inside the file, every entry with dtype / shape / two offsets, known dtype, rank at most 4,
offsets inside the data, byte length equal to numel * element size, no two tensors overlapping.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from ..errors import Corrupt, NotFound, Unsupported

MAX_HEADER_BYTES = 100 << 20
MAX_RANK = 4

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
# dtypes whose header entry is understood but which this engine does not compute with
_KNOWN_UNUSED = {"F64": 8, "I8": 1, "U8": 1, "I16": 2, "U16": 2, "BOOL": 1, "F8_E4M3": 1, "F8_E5M2": 1, "U32": 4, "U64": 8}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafeTensorsFile:
    """A mapped safetensors file; `tensor(name)` returns a CPU tensor that views the mapping."""

    def __init__(self, path: str):
        if not os.path.isfile(path):
            raise NotFound(f"{path}: no such file")
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise Corrupt(f"{path}: too small to hold a safetensors header")
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise Corrupt(f"{path}: header length {hlen} is outside the file")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (ValueError, RecursionError, UnicodeDecodeError) as e:
            raise Corrupt(f"{path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise Corrupt(f"{path}: header is not an object")
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.metadata = header.get("__metadata__", {})
        self.entries: Dict[str, TensorEntry] = {}
        for name, e in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(e, dict) or "dtype" not in e or "shape" not in e or "data_offsets" not in e:
                raise Corrupt(f"{path}: tensor '{name}' lacks dtype, shape or data_offsets")
            dtype, shape, off = e["dtype"], e["shape"], e["data_offsets"]
            if not isinstance(dtype, str) or (dtype not in _DTYPES and dtype not in _KNOWN_UNUSED):
                raise Corrupt(f"{path}: tensor '{name}' has unknown dtype {dtype!r}")
            if (not isinstance(shape, list) or len(shape) > MAX_RANK
                    or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape)):
                raise Corrupt(f"{path}: tensor '{name}' has an invalid shape")
            if (not isinstance(off, list) or len(off) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) for o in off)):
                raise Corrupt(f"{path}: tensor '{name}' has invalid data_offsets")
            begin, end = off
            if begin < 0 or end < begin or end > data_size:
                raise Corrupt(f"{path}: tensor '{name}' lies outside the data")
            elem = _DTYPES[dtype][1] if dtype in _DTYPES else _KNOWN_UNUSED[dtype]
            numel = 1
            for d in shape:
                numel *= d
            if end - begin != numel * elem:
                raise Corrupt(f"{path}: tensor '{name}' has {end - begin} bytes, its shape needs {numel * elem}")
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), begin, end)
        spans = sorted((e.begin, e.end, e.name) for e in self.entries.values() if e.end > e.begin)
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise Corrupt(f"{path}: tensors '{n0}' and '{n1}' overlap")

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries.get(name)
        if e is None:
            raise NotFound(f"{self.path}: no tensor '{name}'")
        if e.dtype not in _DTYPES:
            raise Unsupported(f"{self.path}: tensor '{name}' has dtype {e.dtype}, which this engine cannot execute")
        dtype, elem = _DTYPES[e.dtype]
        numel = (e.end - e.begin) // elem
        if numel == 0:
            return torch.empty(e.shape, dtype=dtype)
        offset = self._data_start + e.begin
        if offset % elem:
            # misaligned data is copied (safetensors.cpp:149-155)
            raw = bytearray(self._map[offset:offset + numel * elem])
            return torch.frombuffer(raw, dtype=dtype, count=numel).reshape(e.shape)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through the view
            t = torch.frombuffer(self._map, dtype=dtype, count=numel, offset=offset)
        return t.reshape(e.shape)

    def close(self) -> None:
        try:
            self._map.close()
        except (BufferError, ValueError):
            pass  # views are still alive; the mapping goes with them
        self._file.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors to `path`, each aligned to 8 bytes."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order: List[Tuple[str, torch.Tensor, int]] = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise Unsupported(f"cannot write tensor '{name}' of dtype {t.dtype}")
        t = t.detach().cpu().contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        order.append((name, t, nbytes))
        offset += nbytes
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for _, t, nbytes in order:
            if nbytes:
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
