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
LONG_SPLIT_KEYS = 4096      # keys per split from which more than CLUSTER_SPLITS splits pay
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

KEY_TILE = 64                 # keys per tile of the tcgen05 prompt attention
PART_MIN_TILES = 24           # fewest key tiles of a part of a query tile (see QueryTileParts)
TILE_PARTS_MAX = 8            # most parts a query tile's keys are dealt into
PART_SLOTS = 64               # records of parts in scratch (one per part of every split tile of a step)
TILE_PARTS = os.environ.get("DYNALM_TILE_PARTS", "1") != "0"      # 0: every query tile walks all of its keys alone


class QueryTileParts:
    """The step plan of the tcgen05 prompt attention: the prompt tiles of QueryTilePlan (without the single-token
    requests at the head of the step, which go to the decode kernel), with the keys of long tiles dealt over several
    entries. A block walks its tile's key tiles one after the other, so a step is as slow as its longest tile, and
    a step with few tiles (a 512-row portion: four per head) leaves most SMs idle however long its context is. With
    the work of all tiles spread evenly over two blocks per SM a block would take `ideal` key tiles; a tile longer
    than 0.6 of that is cut into parts, each at least PART_MIN_TILES key tiles, at most TILE_PARTS_MAX of them, while
    the step's PART_SLOTS records of scratch last (the longest tiles first). A part costs a block's set-up, its record
    in scratch and its share of the merge, so short parts lose. Measured on B200 (32 heads of 64 / of 128, us per
    launch, whole against dealt): 512 rows at 131,072 keys 1,347 -> 877 / 2,060 -> 1,130; at 32,768 keys 343 -> 234 /
    528 -> 300; at 8,192 keys (parts of 31 key tiles) 90 -> 71 / 114 -> 88; at 4,096 keys (parts of 13 to 15) 48 -> 46 /
    62 -> 61; at 2,048 keys (parts of 8 to 10) 28 -> 32 / 34 -> 41; a whole 2,048-token prompt with its eight longest
    tiles in two parts of 9 to 16: 38 -> 48 / 43 -> 60. On the device: int32 [4 + 5 * cap]: a
    header, cap tiles of 4 (as QueryTilePlan's), cap words part | parts << 8 | first record << 16 (0: a whole tile);
    entries with the most key tiles first. What `fill` returns: (entries, records in use, cap)."""

    def __init__(self, n_heads: int, window: int):
        self.n_heads, self.window = int(n_heads), int(window)
        self.name = f"attention_tile_parts:{n_heads}:{window}"

    def ints(self, max_tokens: int, max_requests: int) -> int:
        return 4 + 5 * (max_tokens // Q_TILE + max_requests + PART_SLOTS)

    def key_tiles(self, pos0: int, rows: int) -> int:
        lo = max(0, pos0 - self.window + 1) if self.window > 0 else 0
        return (pos0 + rows - 1) // KEY_TILE - lo // KEY_TILE + 1

    def deal(self, lengths) -> list:
        """Parts per tile for tiles of `lengths` key tiles."""
        slots = 2 * sm_count()
        ideal = sum(lengths) * self.n_heads / slots
        limit = max(0.6 * ideal, float(PART_MIN_TILES))
        parts = [1] * len(lengths)
        left = PART_SLOTS
        for t in sorted(range(len(lengths)), key=lambda t: -lengths[t]):
            want = min(int(-(-lengths[t] // limit)), TILE_PARTS_MAX, lengths[t] // PART_MIN_TILES)
            if want > 1 and want <= left:
                parts[t] = want
                left -= want
        return parts

    def fill(self, host, shape):
        cap = (len(host) - 4) // 5
        lead = 0
        while lead < len(shape.q_len) and shape.q_len[lead] == 1:
            lead += 1
        tiles = []
        for r, (n, r0, start, slot) in enumerate(zip(shape.q_len, shape.q_start, shape.pos_start, shape.slots)):
            if r < lead:
                continue
            for t0 in range(0, n, Q_TILE):
                tiles.append((slot, r0 + t0, min(Q_TILE, n - t0), start + t0))
        lengths = [self.key_tiles(t[3], t[2]) for t in tiles]
        parts = self.deal(lengths) if tiles else []
        entries, record = [], 0
        for t, n_parts in zip(range(len(tiles)), parts):
            per = -(-lengths[t] // n_parts)
            for p in range(n_parts):
                word = 0 if n_parts == 1 else (p | n_parts << 8 | record << 16)
                entries.append((-min(per, lengths[t] - p * per), tiles[t], word))
            if n_parts > 1:
                record += n_parts
        entries.sort(key=lambda e: e[0])
        entries = entries[:cap]
        flat = [v for e in entries for v in e[1]]
        host[4:4 + len(flat)] = flat
        host[4 + 4 * cap:4 + 4 * cap + len(entries)] = [e[2] for e in entries]
        return len(entries), record, cap


_tile_parts = {}


def tile_parts_plan(spec) -> QueryTileParts:
    key = (spec.num_heads, int(spec.get("window", 0)))
    plan = _tile_parts.get(key)
    if plan is None:
        plan = _tile_parts[key] = QueryTileParts(*key)
    return plan

PART_CAP = 32            # most parts a row's keys are cut into
PART_MIN_KEYS = 128      # fewest keys of a part
DECODE_BLOCKS_PER_SM = int(os.environ.get("DYNALM_DECODE_BLOCKS", "2"))     # blocks of the decode kernel that fit an SM
# Whether the keys of a step's single-token rows are dealt into units by the host (DecodeUnits below) instead of every
# row being cut into the same number of parts: 1 always, 0 never, auto (default) from PLANNED_MIN_ROWS rows on. Measured
# on B200: with equal contexts (1B shapes, 2,048 tokens) batch 8 takes 0.925 ms per step planned against 0.900 ms, batch
# 1 gives 1,148 against 1,335 tokens/s (there the parts merge inside a thread-block cluster), batch 64 is equal: with few
# rows the kernel is bound by the latency of a warp's chain of tiles, not by how evenly the blocks are loaded. With
# contexts that differ (continuous batching of the 3B shape, 32 requests of 128 to 4,096 prompt tokens) the decode-only
# step takes 3.63 ms planned against 3.79 ms, the whole run 4,081 against 4,009 tokens/s.
_planned = os.environ.get("DYNALM_DECODE_PLANNED", "auto")
DECODE_PLANNED = _planned != "0"
PLANNED_MIN_ROWS = 1 if _planned == "1" else 12


class DecodeUnits:
    """The step plan of the split-KV decode attention: the keys of the step's single-token requests dealt into units
    of about equal size, about one for every block the GPU can hold at a time, so that a step with one long and many
    short requests, or with few requests, still fills it evenly; a row's share of the units follows its share of the
    keys. On the device: int32 [4 + 4 * units] = (units, 0, 0, 0), then (row, KV-head chunk, part, parts of the row)
    per unit. What `fill` returns: (units, rows). The grid the kernel is launched with depends on the number of rows
    alone (`unit_cap`), so a growing context never changes a CUDA graph."""

    def __init__(self, chunks: int, tile_keys: int, window: int):
        self.chunks, self.tile, self.window = int(chunks), int(tile_keys), int(window)
        self.name = f"attention_decode_units:{chunks}:{tile_keys}:{window}"

    def slots(self) -> int:
        return sm_count() * DECODE_BLOCKS_PER_SM

    def unit_cap(self, rows: int) -> int:
        # one round of blocks, and room for every row to have a part although its share rounds to none
        return self.slots() + rows * self.chunks

    def ints(self, max_tokens: int, max_requests: int) -> int:
        return 4 + 4 * self.unit_cap(max_requests)

    def parts(self, key_counts) -> list:
        """Parts per row for rows that read `key_counts` keys each."""
        rows = len(key_counts)
        tiles = [max(1, -(-n // self.tile)) for n in key_counts]
        budget = self.slots() // self.chunks               # parts over all rows that one round of blocks holds
        if rows >= budget:
            return [1] * rows
        cap = [max(1, min(PART_CAP, n // PART_MIN_KEYS)) for n in key_counts]   # a part keeps a tile for each warp of a block
        total = sum(tiles)
        parts = [max(1, min(cap[r], budget * tiles[r] // total)) for r in range(rows)]
        left = budget - sum(parts)
        while left > 0:
            best, load = -1, 0.0
            for r in range(rows):
                if parts[r] < cap[r] and tiles[r] / parts[r] > load:
                    best, load = r, tiles[r] / parts[r]
            if best < 0:
                break
            parts[best] += 1
            left -= 1
        return parts

    def fill(self, host, shape):
        rows = 0
        while rows < len(shape.q_len) and shape.q_len[rows] == 1:
            rows += 1
        if rows < PLANNED_MIN_ROWS:
            return 0, rows            # few rows: the kernel cuts every row alike (see DECODE_PLANNED)
        counts = [(min(p + 1, self.window) if self.window > 0 else p + 1) for p in shape.pos_start[:rows]]
        parts = self.parts(counts) if rows else []
        flat = [0, 0, 0, 0]
        for r in range(rows):
            for c in range(self.chunks):
                for p in range(parts[r]):
                    flat += (r, c, p, parts[r])
        flat[0] = (len(flat) - 4) // 4
        host[:len(flat)] = flat
        return flat[0], rows


_decode_units = {}


def decode_units_plan(spec) -> DecodeUnits:
    chunks = spec.num_kv_heads * -(-(spec.num_heads // spec.num_kv_heads) // 16)
    key = (chunks, ops.decode_tile_keys(spec.head_dim), int(spec.get("window", 0)))
    plan = _decode_units.get(key)
    if plan is None:
        plan = _decode_units[key] = DecodeUnits(*key)
    return plan


def query_tiles(ctx):
    """(tiles on the device, number of tiles, of prompt tiles, of leading single-token requests) of this step, or
    None when the step was built without the plan."""
    got = ctx.extras.get(QueryTilePlan.name)
    if got is None:
        return None
    return (got[0],) + tuple(got[1])


def decode_splits(rows: int, n_heads: int, n_kv_heads: int, max_kv_len: int, tensor_cores: bool = True,
                  sms: int = 0) -> int:
    """Key splits per row so that the grid fills the GPU, each split at least 128 keys (one tile for each of a
    block's warps: four of 32 keys or eight of 16).

    The tensor-core kernel merges 2, 4 or 8 splits inside a thread-block cluster (no second kernel). Measured on
    B200 (1B shapes, ms per decode step; s = merged by the second kernel): 2,048 keys, batch 1: 4 -> 0.753, 8 ->
    0.741; batch 2: 4 -> 0.758, 8 -> 0.836; batch 4: 4 -> 0.770, 5 -> 0.847, 8 -> 0.921; batch 6: 2 -> 0.821, 4 -> 0.874;
    batch 8: 2 -> 0.832, 3 -> 0.903, 3s -> 0.883, 4 -> 0.881, 4s -> 0.866; 8,192 keys, tokens/s at batch 1: 4 -> 1,171,
    8 -> 1,260, 8s -> 1,131, 16s -> 1,171, 19s -> 1,144; at batch 8: 2 -> 7,423, 3s -> 6,906, 4 -> 7,151, 4s -> 7,070.
    So: a power of two (clusters of 3 or 5 blocks place badly), as many as keep the grid within about one block per
    SM, at most 4 unless there are so few rows that 8 still leaves SMs free. Only from 32,768 keys on are more
    splits taken, merged by the second kernel."""
    group = n_heads // n_kv_heads
    blocks = rows * n_kv_heads * (-(-group // (16 if tensor_cores else 4)))
    sms = sms or sm_count()
    want = -(-DECODE_FILL * sms // max(blocks, 1))
    most = max(1, max_kv_len // 128)
    if not tensor_cores:
        return max(1, min(want, most, MAX_SPLITS))
    if want > CLUSTER_SPLITS and max_kv_len >= CLUSTER_SPLITS * LONG_SPLIT_KEYS:
        return max(1, min(want, most, MAX_SPLITS))
    cap = CLUSTER_SPLITS if blocks * CLUSTER_SPLITS <= sms // 2 else 4
    splits = 1
    while splits * 2 <= min(cap, most) and blocks * splits * 2 * 4 <= 5 * DECODE_FILL * sms:
        splits *= 2
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
    planned = ctx.extras.get(decode_units_plan(spec).name) if (DECODE_PLANNED and decode_uses_tensor_cores(spec)
                                                              and qkv.stride(0) % 8 == 0) else None
    if planned is not None and planned[1][1] == rows and planned[1][0] > 0:
        plan = decode_units_plan(spec)
        most_rows = max(runtime.max_requests, rows)
        scratch = runtime.flat(f"attn_split_scratch_{spec.num_heads}x{spec.head_dim}",
                               ops.decode_scratch_floats(most_rows, spec.num_heads, spec.head_dim, MAX_SPLITS))
        counters = runtime.flat(f"attn_unit_counters_{plan.chunks}", most_rows * plan.chunks, torch.int32)
        ops.paged_attention_decode_planned(qkv[:rows], k_cache, v_cache, cache.block_table, ctx.positions[:rows],
                                           ctx.row_slot[:rows], out[:rows], scratch, counters, planned[0],
                                           plan.unit_cap(rows), PART_CAP, spec.num_heads, spec.num_kv_heads, spec.head_dim,
                                           cache.page_size, float(spec.scale), spec.get("window", 0))
        return
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
        tcgen05 = use_prefill_tcgen05(spec, qkv, out, cache.page_size)
        dealt = ctx.extras.get(tile_parts_plan(spec).name) if (tcgen05 and TILE_PARTS) else None
        if dealt is not None and dealt[1][1] > 0:
            # some tiles' keys are dealt over several blocks: the plan's own list of entries, and scratch for the parts
            view, (entries, records, cap) = dealt
            partial = runtime.flat(f"attn_tile_parts_{spec.num_heads}x{spec.head_dim}",
                                   PART_SLOTS * spec.num_heads * (spec.head_dim + 2) * Q_TILE, torch.float32)
            counters = runtime.flat(f"attn_tile_part_counters_{spec.num_heads}", PART_SLOTS * spec.num_heads, torch.int32)
            ops.paged_attention_prefill_tcgen05(qkv, k_cache, v_cache, cache.block_table, view[4:4 + 4 * cap], entries, out,
                                                spec.num_heads, spec.num_kv_heads, spec.head_dim, cache.page_size,
                                                float(spec.scale), spec.get("window", 0),
                                                unit_parts=view[4 + 4 * cap:4 + 5 * cap], partial=partial, counters=counters)
        else:
            kernel = ops.paged_attention_prefill_tcgen05 if tcgen05 else ops.paged_attention_prefill
            kernel(qkv, k_cache, v_cache, cache.block_table, q_tiles, n_tiles, out, spec.num_heads,
                   spec.num_kv_heads, spec.head_dim, cache.page_size, float(spec.scale), spec.get("window", 0))
    if side is not None:
        ops.stream_join(side)
    return True
