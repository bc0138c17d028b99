"""From a model folder (or a configuration and tensors in memory) to a ready step function."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch

from .. import models  # noqa: F401  (registers the architectures)
from .. import parts  # noqa: F401   (registers the part kinds)
from ..cache import DEFAULT_PAGE_SIZE, CacheManager
from ..errors import InvalidArgument
from ..registry import find_architecture
from ..weights.loader import check_tensors, open_model_folder, place_tensors
from . import memory
from .model import Decoder
from .runtime import Runtime, parse_dtype
from .step import StepFunction


@dataclass
class BuiltModel:
    config: Any
    plan: Any
    runtime: Runtime
    model: Decoder
    cache: CacheManager
    step_fn: StepFunction


def build(model_dir: Optional[str] = None, *, config_obj: Optional[Mapping[str, Any]] = None,
          tensors: Optional[Mapping[str, torch.Tensor]] = None, dtype="bfloat16", kv_tokens: Optional[int] = None,
          max_batch_tokens: int = 2048, max_requests: int = 64, page_size: int = DEFAULT_PAGE_SIZE,
          device="cuda:0", context: Optional[int] = None) -> BuiltModel:
    """Load weights, build the model and its cache.

    model_dir          a folder with config.json and model.safetensors, or
    config_obj+tensors a config.json dict and CPU tensors by file name (random-weights mode without a file)
    kv_tokens          tokens the cache pool holds over all live requests (default: sized from the device memory that
                       is free after the weights, engine/memory.py); a size that cannot fit is refused before
                       anything is allocated, with the largest size that would fit
    max_batch_tokens   the most tokens one step may bring
    context            the longest one request may grow (default: max_position_embeddings)
    """
    compute = parse_dtype(dtype)
    runtime = Runtime(device, compute, max_tokens=max_batch_tokens, max_requests=max_requests)
    free_before = torch.cuda.mem_get_info(runtime.device)[0]
    if model_dir is not None:
        folder = open_model_folder(model_dir)
        config, plan = folder.config, folder.plan
        store = place_tensors(plan, folder, runtime.device, compute)
        folder.close()
    else:
        if config_obj is None or tensors is None:
            raise InvalidArgument("build needs a model folder, or a configuration and its tensors")
        arch = find_architecture(config_obj)
        config = arch.read_config(config_obj)
        plan = arch.plan(config, present=set(tensors))
        check_tensors("tensors", plan, {n: tuple(t.shape) for n, t in tensors.items()})
        store = place_tensors(plan, tensors, runtime.device, compute)
    model = Decoder(plan, store, runtime)
    ctx_len = int(context or plan.context_length)
    specs = model.cache_specs()
    per_token = memory.cache_bytes_per_token(specs, 2 if compute == torch.bfloat16 else 4)
    weights = model.weight_bytes()
    kv = int(kv_tokens) if kv_tokens else memory.auto_kv_tokens(ctx_len, per_token, weights, free_before)
    pages = -(-kv // page_size)
    memory.check_memory_fit(weights, pages * page_size * per_token, per_token, free_before)
    cache = CacheManager(specs, page_size, kv, max_requests, ctx_len, runtime.device, compute)
    step_fn = StepFunction(model, cache, runtime, max_requests)
    if compute == torch.bfloat16:
        # the library product that a few shapes still go to (kernels/gemm.py) sets itself up at its first call, which
        # takes about 140 ms: here, not inside the first request
        warm = torch.zeros(32, 64, dtype=compute, device=runtime.device)
        torch.mm(warm, warm.t())
    return BuiltModel(config, plan, runtime, model, cache, step_fn)
