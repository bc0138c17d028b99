"""How large the cache may be, decided before it is allocated.

The reference sizes its KV cache from the memory left after the weights when the user gives no size
(`auto_kv_tokens`, dynalm/src/runtime/engine.cpp:96-104) and refuses a configuration that cannot fit at load
time with a message that says what would (`check_memory_fit`, engine.cpp:120-145), instead of failing inside the
first large allocation. The same two decisions, for one GPU.
"""

from __future__ import annotations

from typing import Optional, Sequence

from ..errors import ResourceExhausted

BLOCK = 16
AUTO_MAX_TOKENS = 65536
AUTO_FLOOR_TOKENS = 2048
USABLE_PERCENT = 95            # of the device memory that was free before the model was loaded


def cache_bytes_per_token(specs: Sequence[Optional[object]], compute_itemsize: int) -> int:
    """Bytes of cache one token takes over all run-order entries that keep pages (`specs`: their CacheSpecs)."""
    total = 0
    for s in specs:
        if s is None or s.kind != "pages":
            continue
        n = 1
        for d in s.entry_shape:
            n *= int(d)
        item = {"float32": 4, "bfloat16": 2, None: compute_itemsize}[s.dtype]
        total += s.tensors * n * item
    return total


def auto_kv_tokens(context_length: int, per_token: int, weight_bytes: int, available: int) -> int:
    """Tokens of cache when the user gave none: half of what is left of `available` after the weights, at most
    65,536 tokens, at least min(context, 2,048), in whole blocks of 16."""
    if available <= 0:
        return min(int(context_length), 16384)
    per_token = max(1, int(per_token))
    budget = max(0, int(available) - int(weight_bytes)) // 2
    floor = min(int(context_length), AUTO_FLOOR_TOKENS)
    tokens = min(max(budget // per_token, floor), max(floor, AUTO_MAX_TOKENS))
    return max(BLOCK, tokens // BLOCK * BLOCK)


def _gib(b: int) -> str:
    mib = int(b) // (1 << 20)
    return f"{mib // 1024}.{mib % 1024 * 10 // 1024} GiB"


def check_memory_fit(weight_bytes: int, kv_bytes: int, kv_per_token: int, device_free: int,
                     workspace_bytes: int = 0) -> None:
    """Raise ResourceExhausted, with the largest --ctx that would fit, when weights + cache (+ workspace) exceed 95 %
    of the device memory that was free before loading. `device_free` < 0: not known, nothing is checked."""
    if device_free < 0:
        return
    limit = int(device_free) // 100 * USABLE_PERCENT
    need = int(weight_bytes) + int(kv_bytes) + int(workspace_bytes)
    if need <= limit:
        return
    fit = max(0, limit - int(weight_bytes) - int(workspace_bytes)) // max(1, int(kv_per_token)) // BLOCK * BLOCK
    msg = (f"not enough GPU memory: the model needs {_gib(weight_bytes)} and the KV cache {_gib(kv_bytes)}, "
           f"{_gib(need)} in all; the limit is {_gib(limit)}")
    msg += (f"; use --ctx {fit} or less" if fit >= BLOCK
            else "; this model does not fit, use a smaller model")
    raise ResourceExhausted(msg)
