"""Device time per kernel of steps that run launch by launch.

`kernel_times(step_fn)` is a context manager: inside it the step function replays no CUDA graph, every layer
goes through its parts (no list of launches issued by address), the attention kernels of a mixed step run one after
the other, and every launch stands between two CUDA events (`ops.KernelTimes`). The times are those of kernels
that do not overlap their neighbours, so they add up to more than the step takes in service; they say where
the time goes. `DYNALM_FORWARD_PROFILE=1 dynalm run ...` prints the table after a generation.

The reference marks its forward pass per op with wall-clock times, off by default (`ForwardProfile`,
dynalm/src/model/transformer.h:34-49, transformer.cpp:479-484).
"""

from __future__ import annotations

import contextlib
from typing import Dict, Tuple

from ..kernels import attention, ops
from . import launch_memo


@contextlib.contextmanager
def kernel_times(step_fn):
    saved = (step_fn.use_graphs, launch_memo.ENABLED, attention.SIDE_BY_SIDE)
    step_fn.use_graphs, launch_memo.ENABLED, attention.SIDE_BY_SIDE = False, False, False
    try:
        with ops.KernelTimes() as times:
            yield times
    finally:
        step_fn.use_graphs, launch_memo.ENABLED, attention.SIDE_BY_SIDE = saved


def table(totals: Dict[str, Tuple[int, float]]) -> str:
    """The totals as lines, the longest first."""
    whole = sum(ms for _, ms in totals.values()) or 1.0
    lines = [f"{'kernel':40s} {'launches':>8s} {'ms':>10s} {'share':>6s}"]
    for name, (n, ms) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{name:40s} {n:8d} {ms:10.3f} {100.0 * ms / whole:5.1f}%")
    return "\n".join(lines)
