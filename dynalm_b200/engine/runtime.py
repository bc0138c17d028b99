"""What every part is built with: the device, the compute dtype and a workspace of named buffers."""

from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..errors import ExtensionMissing, InvalidArgument, Unsupported


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.float32, torch.bfloat16):
            return name
        raise Unsupported(f"compute dtype {name} is not supported (float32 and bfloat16 are)")
    table = {"float32": torch.float32, "f32": torch.float32, "fp32": torch.float32,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    try:
        return table[str(name).lower()]
    except KeyError:
        raise InvalidArgument(f"unknown dtype '{name}' (float32 or bfloat16)") from None


class Runtime:
    """Device, dtype and scratch memory shared by the parts of one model.

    `buffer(name, shape, dtype)` hands out a persistent tensor: the same name and trailing shape
    give the same storage every step (so pointers stay fixed for CUDA-graph replay), sized for
    `max_tokens` rows and sliced to the rows asked for. Two parts that use the same name and width
    share the storage; that is safe because a buffer's contents never outlive the part call that
    filled it, except where a name says otherwise.
    """

    def __init__(self, device="cuda:0", dtype="bfloat16", max_tokens: int = 2048, max_requests: int = 64):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ExtensionMissing("dynalm_b200 runs on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise ExtensionMissing("no CUDA device is available; dynalm_b200 has no CPU path")
        self.dtype = parse_dtype(dtype)
        self.max_tokens = int(max_tokens)
        self.max_requests = int(max_requests)      # the most rows a decode-only step can bring
        self._buffers: Dict[Tuple, torch.Tensor] = {}
        self._views: Dict[Tuple, torch.Tensor] = {}      # (name, shape, dtype) -> the first rows of a buffer
        self._side_stream = None

    @property
    def side_stream(self) -> int:
        """The handle of a second stream, for a kernel that may run beside the kernels of the step's own stream
        (ops.stream_fork / ops.stream_join put it in order)."""
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        return self._side_stream.cuda_stream

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype = None) -> torch.Tensor:
        dtype = dtype or self.dtype
        view = self._views.get((name, shape, dtype))
        if view is not None:
            return view
        rows, tail = int(shape[0]), tuple(int(s) for s in shape[1:])
        if rows > self.max_tokens:
            raise InvalidArgument(f"{rows} rows asked of buffer '{name}', the runtime was made for {self.max_tokens}")
        key = (name, tail, dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros((self.max_tokens,) + tail, dtype=dtype, device=self.device)
            self._buffers[key] = buf
        view = buf[:rows]
        if isinstance(shape, tuple):
            self._views[(name, shape, dtype)] = view
        return view

    def flat(self, name: str, numel: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """A persistent 1-D scratch array of `numel` elements, allocated once at the size first asked
        for (callers ask for their maximum), so that its address never changes."""
        key = (name, "flat", dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.zeros(int(numel), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        if buf.numel() < numel:
            raise InvalidArgument(f"scratch '{name}' was made for {buf.numel()} elements, {numel} are asked for")
        return buf

    def workspace_bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
