"""Sizing the cache and refusing what cannot fit (engine/memory.py), with made-up memory figures."""

import pytest

from dynalm_b200.engine import memory
from dynalm_b200.errors import ResourceExhausted
from dynalm_b200.parts.base import CacheSpec

GIB = 1 << 30


def test_bytes_per_token_counts_pages_only():
    specs = [CacheSpec("pages", (8, 64)), None, CacheSpec("pages", (8, 64), dtype="float32"),
             CacheSpec("state", state_shape=(4, 4)), CacheSpec("pages", (2, 16), tensors=1, window=32)]
    assert memory.cache_bytes_per_token(specs, 2) == 2 * 8 * 64 * 2 + 2 * 8 * 64 * 4 + 2 * 16 * 2
    # the Llama 3.2 1B shape in bfloat16: 32 KiB a token
    assert memory.cache_bytes_per_token([CacheSpec("pages", (8, 64))] * 16, 2) == 32 * 1024


def test_auto_size_follows_the_reference_rule():
    per_token = 32 * 1024
    # half of what is left after the weights, in whole blocks
    assert memory.auto_kv_tokens(8192, per_token, 2 * GIB, 3 * GIB) == (GIB // 2) // per_token // 16 * 16
    # capped at 65,536 tokens however much memory there is
    assert memory.auto_kv_tokens(131072, per_token, 2 * GIB, 180 * GIB) == 65536
    # never below min(context, 2048), even when nothing is left (the fit check then refuses)
    assert memory.auto_kv_tokens(8192, per_token, 4 * GIB, 3 * GIB) == 2048
    assert memory.auto_kv_tokens(512, per_token, 4 * GIB, 3 * GIB) == 512
    # memory not known
    assert memory.auto_kv_tokens(8192, per_token, 2 * GIB, 0) == 8192
    assert memory.auto_kv_tokens(131072, per_token, 2 * GIB, -1) == 16384


def test_fit_check_names_the_size_that_would_fit():
    per_token = 128 * 1024
    free = 10 * GIB
    memory.check_memory_fit(4 * GIB, 4 * GIB, per_token, free)               # 8 of 9.5 GiB
    memory.check_memory_fit(40 * GIB, 400 * GIB, per_token, -1)              # memory not known: not checked
    with pytest.raises(ResourceExhausted) as e:
        memory.check_memory_fit(4 * GIB, 8 * GIB, per_token, free)
    msg = str(e.value)
    assert "not enough GPU memory: the model needs 4.0 GiB and the KV cache 8.0 GiB, 12.0 GiB in all" in msg
    limit = free // 100 * 95
    fit = (limit - 4 * GIB) // per_token // 16 * 16
    assert f"use --ctx {fit} or less" in msg
    memory.check_memory_fit(4 * GIB, fit * per_token, per_token, free)        # and that size does fit
    with pytest.raises(ResourceExhausted, match="this model does not fit"):
        memory.check_memory_fit(12 * GIB, 1 * GIB, per_token, free)
