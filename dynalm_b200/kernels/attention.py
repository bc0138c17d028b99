"""Chooses the attention kernel for a step.

float32 always runs the plain kernel (csrc/attention_generic.cu), whose arithmetic for a row is
fixed by the row alone. bfloat16 steps in which every request brings one token run the split-KV
kernel (csrc/attention_decode.cu); other bfloat16 steps (prompt portions, alone or beside decode
rows) run a flash kernel: the tcgen05 one (csrc/attention_prefill_tcgen05.cu) for head sizes 64 and
128 with pages of at least 16 keys, else the mma.sync one (csrc/attention_prefill.cu). Every shape
the faster kernels refuse falls to the plain kernel.
"""

from __future__ import annotations

import os

import torch

from . import ops

from .device import sm_count

MAX_SPLITS = 32
CLUSTER_SPLITS = 8          # up to here the tensor-core kernel merges splits inside a thread-block cluster
LONG_SPLIT_KEYS = 1024      # keys per split from which more than CLUSTER_SPLITS splits pay
DECODE_FILL = int(os.environ.get('DYNALM_DECODE_FILL', '1'))   # blocks per SM the split count aims for


Q_TILE = 128      # query rows of one request per tile: the row block of the tcgen05 prompt kernel


class QueryTilePlan:
    """The step plan of the prompt attention kernels: every request of the step cut into tiles of at most Q_TILE
    consecutive rows, int32 [tiles, 4] = (request slot, first row of the step, rows, first position). The tiles of
    prompt portions come first, those that read the most keys first (the attention grid then ends evenly); then the
    one-row tiles of the requests at the head of the step that bring a single token each: a mixer hands those rows
    to its decode kernel and only the first `prompt_tiles` tiles to its prompt kernel. What `fill` returns:
    (tiles, prompt_tiles, leading single-token requests)."""

    name = "attention_query_tiles"

    def ints(self, max_tokens: int, max_requests: int) -> int:
        return 4 * (max_tokens // Q_TILE + max_requests)

    def fill(self, host, shape):
        lead = 0
        while lead < len(shape.q_len) and shape.q_len[lead] == 1:
            lead += 1
        tiles = []
        for r, (n, r0, start, slot) in enumerate(zip(shape.q_len, shape.q_start, shape.pos_start, shape.slots)):
            for t0 in range(0, n, Q_TILE):
                tiles.append((r >= lead, -(start + t0 + min(Q_TILE, n - t0)), slot, r0 + t0, min(Q_TILE, n - t0), start + t0))
        tiles.sort(key=lambda t: (not t[0], t[1]))
        flat = [v for t in tiles for v in t[2:]]
        host[:len(flat)] = flat
        return len(tiles), len(tiles) - lead, lead


QUERY_TILES = QueryTilePlan()


def query_tiles(ctx):
    """(tiles on the device, number of tiles, of prompt tiles, of leading single-token requests) of this step, or
    None when the step was built without the plan."""
    got = ctx.extras.get(QueryTilePlan.name)
    if got is None:
        return None
    return (got[0],) + tuple(got[1])


def decode_splits(rows: int, n_heads: int, n_kv_heads: int, max_kv_len: int, tensor_cores: bool = True,
                  sms: int = 0) -> int:
    """Key splits per row so that the grid fills the GPU, each split at least 128 keys (one 32-key tile for each
    of a block's four warps). The tensor-core kernel merges up to 8 splits inside a thread-block cluster, which
    wins while a split is short; from 1,024 keys per split on, more splits (merged by a second kernel) win."""
    group = n_heads // n_kv_heads
    blocks = rows * n_kv_heads * (-(-group // (16 if tensor_cores else 4)))
    want = -(-DECODE_FILL * (sms or sm_count()) // max(blocks, 1))
    splits = max(1, min(want, max(1, max_kv_len // 128), MAX_SPLITS))
    if tensor_cores and splits > CLUSTER_SPLITS and max_kv_len < CLUSTER_SPLITS * LONG_SPLIT_KEYS:
        splits = CLUSTER_SPLITS
    return splits


def decode_uses_tensor_cores(spec) -> bool:
    return spec.head_dim <= 128


def decode_plan(ctx, spec, rows: int = 0) -> int:
    """The number of key splits for the step's decode rows (all rows unless `rows` says how many); also part
    of the CUDA-graph key."""
    span = ctx.max_kv_len if spec.get("window", 0) <= 0 else min(ctx.max_kv_len, spec.get("window", 0))
    # bucket the span so that a growing context changes the launch shape only now and then
    bucket = 256
    while bucket < span:
        bucket *= 2
    return decode_splits(rows or ctx.num_tokens, spec.num_heads, spec.num_kv_heads, bucket, decode_uses_tensor_cores(spec))


SIDE_BY_SIDE = os.environ.get("DYNALM_ATTENTION_SIDE_BY_SIDE", "1") != "0"    # 0: the two attention kernels of a mixed step one after the other
MIXED_DECODE_ROWS = 1      # from this many leading decode rows on, a mixed step runs them through the decode kernel


def decode_kernel_takes(spec, dtype: torch.dtype, page_size: int) -> bool:
    return dtype == torch.bfloat16 and page_size & (page_size - 1) == 0 and spec.head_dim % 16 == 0 and spec.head_dim <= 256


def use_decode_kernel(ctx, spec, dtype: torch.dtype, page_size: int) -> bool:
    return ctx.decode_only and decode_kernel_takes(spec, dtype, page_size)


def use_prefill_kernel(ctx, spec, qkv: torch.Tensor, page_size: int) -> bool:
    return (qkv.dtype == torch.bfloat16 and query_tiles(ctx) is not None and page_size & (page_size - 1) == 0
            and spec.head_dim % 16 == 0 and spec.head_dim <= 128 and qkv.stride(0) % 8 == 0)


PREFILL_TCGEN05 = os.environ.get("DYNALM_PREFILL_TCGEN05", "1") != "0"     # 0: the mma.sync kernel for every head size


def use_prefill_tcgen05(spec, qkv: torch.Tensor, out: torch.Tensor, page_size: int) -> bool:
    return (PREFILL_TCGEN05 and spec.head_dim in ops.PREFILL_TCGEN05_HEAD_DIMS and page_size >= 16
            and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0 and qkv.data_ptr() % 16 == 0)


def _decode_rows(qkv: torch.Tensor, cache, ctx, out: torch.Tensor, spec, runtime, rows: int) -> None:
    """The split-KV kernel on rows 0 .. rows - 1 (each the newest token of its request)."""
    k_cache, v_cache = cache.arrays
    n_split = decode_plan(ctx, spec, rows)
    scratch = None
    if n_split > 1:
        most_rows = max(runtime.max_requests, rows)
        scratch = runtime.flat(f"attn_split_scratch_{spec.num_heads}x{spec.head_dim}",
                               ops.decode_scratch_floats(most_rows, spec.num_heads, spec.head_dim, MAX_SPLITS))
    ops.paged_attention_decode(qkv[:rows], k_cache, v_cache, cache.block_table, ctx.positions[:rows], ctx.row_slot[:rows],
                               out[:rows], scratch, spec.num_heads, spec.num_kv_heads, spec.head_dim, cache.page_size,
                               float(spec.scale), spec.get("window", 0), n_split,
                               tensor_cores=decode_uses_tensor_cores(spec) and qkv.stride(0) % 8 == 0)


def paged_attention(qkv: torch.Tensor, cache, ctx, out: torch.Tensor, spec, runtime) -> bool:
    """Run the fast kernel(s) for this step if they apply; False means the caller runs the plain one."""
    k_cache, v_cache = cache.arrays
    if use_decode_kernel(ctx, spec, qkv.dtype, cache.page_size):
        _decode_rows(qkv, cache, ctx, out, spec, runtime, qkv.shape[0])
        return True
    if not use_prefill_kernel(ctx, spec, qkv, cache.page_size):
        return False
    q_tiles, n_tiles, n_prompt_tiles, leading = query_tiles(ctx)
    side = None
    if leading >= MIXED_DECODE_ROWS and decode_kernel_takes(spec, qkv.dtype, cache.page_size):
        # a mixed step: the decode rows at its head go through the split-KV kernel (as a one-row query tile each
        # of them would occupy a whole block of the prompt kernel), the prompt portions through the flash kernel.
        # The two kernels read and write different rows and each fills a part of the GPU only: they run side by side,
        # the decode rows on a second stream.
        n_tiles = n_prompt_tiles
        if SIDE_BY_SIDE and n_tiles > 0:
            side = runtime.side_stream
            ops.stream_fork(side)
            with ops.on_stream(side):
                _decode_rows(qkv, cache, ctx, out, spec, runtime, leading)
        else:
            _decode_rows(qkv, cache, ctx, out, spec, runtime, leading)
    if n_tiles > 0:
        kernel = (ops.paged_attention_prefill_tcgen05 if use_prefill_tcgen05(spec, qkv, out, cache.page_size)
                  else ops.paged_attention_prefill)
        kernel(qkv, k_cache, v_cache, cache.block_table, q_tiles, n_tiles, out, spec.num_heads,
               spec.num_kv_heads, spec.head_dim, cache.page_size, float(spec.scale), spec.get("window", 0))
    if side is not None:
        ops.stream_join(side)
    return True
