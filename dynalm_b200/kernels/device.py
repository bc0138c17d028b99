"""What the dispatchers need to know of the device they size grids for."""

from __future__ import annotations

from typing import Dict

import torch

_sm: Dict[int, int] = {}
B200_SMS = 148


def sm_count(device=None) -> int:
    """Multiprocessors of `device` (the current CUDA device when None), read from the driver once per device; where
    there is no CUDA device (the dispatch rules are tested on the CPU) the B200's 148."""
    if not torch.cuda.is_available():
        return B200_SMS
    index = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    got = _sm.get(index)
    if got is None:
        got = torch.cuda.get_device_properties(index).multi_processor_count
        _sm[index] = got
    return got
