"""Layers of equal structure launch the same kernels: issue them once from Python, then again by address.

Within one step every layer of a model with equal parts runs the same sequence of kernel launches with the same
arguments, except for the addresses of the layer's own tensors (its weights, its pages of the cache). The Python
path from a block's `forward` down to a launch (choice of kernel, checks, scratch lookups) costs far more than
the launch, and a step that is not replayed from a CUDA graph (every step with a prompt portion in it) pays it
for every layer. So the first layer of a kind is run through Python with its launches written down (the C entry
point and its arguments, `ops.Recording`), and the layers after it re-issue that list with the addresses of
their own tensors put in place of the first layer's.

What makes this safe:

* only blocks whose parts all say `replay_safe` take part: all their device work goes through the recorded C
  calls, and depends only on the step, the block's inputs and the part's own tensors. A part defined elsewhere
  (a test's toy mixer) does not say so and always runs through its own `forward`;
* a list is reused only by a layer with the same block class and spec, the same state of the residual stream on
  entry (what is pending, where, at what scale), and tensors of the same shapes, dtypes, strides and 16-byte
  alignment in the same order;
* every argument that points into one of the recorded layer's tensors is moved to the same offset of the other
  layer's tensor (a library product is written down with its tensors, and the layer's own tensor among them is
  exchanged); all other arguments (shared scratch, the step's index arrays, sizes) stay.

The addresses of a layer's tensors are read once, at the layer's first step, and kept by the model
(`Decoder._run_layouts`): a part's tensors may be changed in place afterwards, but a part that gets another tensor
object must be followed by `Decoder.forget_layouts()`.

The reference has no counterpart: its layer loop is compiled C++ (dynalm/src/model/transformer.cpp:596-699).
"""

from __future__ import annotations

import bisect
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..errors import EngineError
from ..kernels import gemm, ops

ENABLED = os.environ.get("DYNALM_LAYER_REPLAY", "1") != "0"     # 0: every layer through its parts' Python code
REPLAYED_LAYERS = 0          # layers issued from a list so far


def owned_tensors(obj, depth: int = 0) -> List[torch.Tensor]:
    """The tensors a block and its parts hold, in an order that is the same for two objects built by the same code.
    A part may say so itself (`replay_tensors() -> list`); else its attributes are walked in order: tensors, and
    objects that are parts in their own right (they say `replay_safe` of themselves, wherever their class lives)."""
    own = getattr(obj, "replay_tensors", None)
    if own is not None:
        return list(own())
    found: List[torch.Tensor] = []
    for name, value in vars(obj).items():
        if isinstance(value, torch.Tensor):
            found.append(value)
        elif depth < 3 and hasattr(value, "__dict__") and hasattr(value, "replay_safe"):
            found.extend(owned_tensors(value, depth + 1))
    return found


class _Layout:
    """A layer's tensors as the recorded calls see them: addresses, sizes, and what must agree between two layers."""

    __slots__ = ("tensors", "pointers", "sizes", "signature")
    _interned: Dict[tuple, int] = {}

    def __init__(self, tensors: List[torch.Tensor]):
        self.tensors = tensors
        self.pointers = [t.data_ptr() for t in tensors]
        self.sizes = [t.numel() * t.element_size() if t.is_contiguous() else
                      (sum((n - 1) * s for n, s in zip(t.shape, t.stride())) + 1) * t.element_size() for t in tensors]
        described = tuple((tuple(t.shape), t.dtype, t.stride(), t.data_ptr() & 15) for t in tensors)
        self.signature = self._interned.setdefault(described, len(self._interned))      # a small number per layout


class _Record:
    __slots__ = ("calls", "own", "library", "pending", "pending_scale")

    def __init__(self, calls, pending, pending_scale):
        # [(function, arguments, ((argument index, tensor index, offset or None for the tensor itself), ...))]
        self.calls = calls
        self.library = sum(1 for f, _, _ in calls if f is ops.library_mm_again)
        self.own = sum(1 for f, _, _ in calls if ops.counts_as_kernel(f))
        self.pending = pending
        self.pending_scale = pending_scale


def _patches(calls, layout: _Layout):
    """For every recorded call, which arguments point into which of the layer's tensors."""
    order = sorted(range(len(layout.pointers)), key=lambda j: layout.pointers[j])
    starts = [layout.pointers[j] for j in order]
    out = []
    for f, args in calls:
        patch = []
        for idx, a in enumerate(args):
            if type(a) is int and a >= 4096:
                k = bisect.bisect_right(starts, a) - 1
                if k >= 0:
                    j = order[k]
                    if a - layout.pointers[j] < layout.sizes[j]:
                        patch.append((idx, j, a - layout.pointers[j]))
            elif isinstance(a, torch.Tensor):
                for j, t in enumerate(layout.tensors):
                    if t.data_ptr() == a.data_ptr() and t.shape == a.shape and t.stride() == a.stride():
                        patch.append((idx, j, None))
                        break
        out.append((f, args, tuple(patch)))
    return out


class LayerLaunchMemo:
    """One step's lists of launches, by kind of layer. `layouts` (run-order entry -> _Layout) and `kinds` outlive
    the step; the model keeps them."""

    def __init__(self, layouts: Dict[int, Tuple[object, _Layout]], kinds: List[int]):
        self.layouts = layouts
        self.kinds = kinds                  # run-order entry -> a number that blocks of equal class and spec share
        self.records: Dict[tuple, Optional[_Record]] = {}

    def _layout(self, index: int, block, cache) -> _Layout:
        got = self.layouts.get(index)
        if got is None or got[0] is not cache:             # the view is kept, so that no other object can take its place
            tensors = owned_tensors(block)
            if cache is not None:
                tensors = tensors + list(cache.arrays) + ([cache.block_table] if cache.block_table is not None else [])
            got = (cache, _Layout(tensors))
            self.layouts[index] = got
        return got[1]

    def run(self, index: int, block, stream, ctx, cache, owns_cache: bool):
        if not getattr(block, "replay_safe", False):
            return block.forward(stream, ctx, cache, owns_cache)
        layout = self._layout(index, block, cache)
        pending = stream.pending
        key = (self.kinds[index], owns_cache, stream.x.data_ptr(), stream.pending_scale,
               None if pending is None else (pending.data_ptr(), tuple(pending.shape), pending.dtype), layout.signature)
        if key in self.records:
            record = self.records[key]
            if record is None:
                return block.forward(stream, ctx, cache, owns_cache)
            pointers, tensors = layout.pointers, layout.tensors
            for f, args, patch in record.calls:
                if patch:
                    args = list(args)
                    for idx, j, offset in patch:
                        args[idx] = tensors[j] if offset is None else pointers[j] + offset
                code = f(*args)
                if code != 0:
                    raise EngineError(f"a replayed launch of layer {index} failed: CUDA error {code}")
            ops.LAUNCHES += record.own
            gemm.LIBRARY_CALLS += record.library
            global REPLAYED_LAYERS
            REPLAYED_LAYERS += 1
            stream.pending, stream.pending_scale = record.pending, record.pending_scale
            return stream
        with ops.Recording() as recording:
            stream = block.forward(stream, ctx, cache, owns_cache)
        if any(f is None for f, _ in recording.calls):
            self.records[key] = None             # some work was not written down: this kind runs through its parts
        else:
            self.records[key] = _Record(_patches(recording.calls, layout), stream.pending, stream.pending_scale)
        return stream
