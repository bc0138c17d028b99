"""Which kernel a matrix product and a decode attention go to, by shape: the decisions of kernels/gemm.py and
kernels/attention.py on tensors that are never touched (no GPU needed)."""

import os

import torch

from dynalm_b200.kernels import attention, gemm


def _xw(rows, n, k, dtype=torch.bfloat16):
    return torch.zeros(rows, k, dtype=dtype), torch.zeros(n, k, dtype=dtype)


def test_few_rows_go_to_the_weight_streaming_products():
    for rows in (1, 8):
        x, w = _xw(rows, 2048, 2048)
        assert gemm.skinny_ok(x, w) and not gemm.use_stream(x, w)          # mma.sync up to 8 rows
    for rows in (9, 16):
        x, w = _xw(rows, 2048, 2048)
        assert gemm.use_stream(x, w)                                        # tcgen05, computed transposed, 9 to 16
    x, w = _xw(17, 2048, 2048)
    assert not gemm.use_stream(x, w) and not gemm.skinny_ok(x, w)
    # a K that is no multiple of 8, or float32, takes neither
    x, w = _xw(4, 256, 100)
    assert not gemm.skinny_ok(x, w) and not gemm.use_stream(x, w)
    x, w = _xw(12, 256, 128, torch.float32)
    assert not gemm.skinny_ok(x, w) and not gemm.use_stream(x, w)


def test_k_splits_fill_the_gpu_but_stay_few():
    # o and down of the 1B shape at 9 to 16 rows: 16 feature tiles, at most 6 splits, each of at least 256 of K
    assert gemm.stream_split_count(2048, 2048) == 6
    assert gemm.stream_split_count(2048, 8192) == 6
    assert gemm.stream_split_count(2048, 512) == 2
    assert gemm.stream_split_count(128256, 2048) == 1
    # the mma.sync kernel: up to 8 blocks along K, none for a wide output
    assert gemm.split_count(2048, 2048, 8) == 3
    assert gemm.split_count(16384, 2048, 8) == 1


def test_the_tcgen05_product_needs_96_tiles_at_its_narrowest_width():
    def ok(rows, n, k=2048):
        x, w = _xw(rows, n, k)
        return gemm.tcgen05_ok(x, w, torch.zeros(rows, n, dtype=torch.bfloat16), n)
    assert ok(2048, 2048) and ok(2048, 16384)
    assert ok(544, 3072)                    # 5 row blocks x 24 tiles of 128: a 512-token portion's O and down
    assert not ok(64, 2048)                 # a decode batch of 64: the library's split-K kernel
    assert ok(17, 128256)                   # the vocabulary product from 17 rows
    assert not ok(2048, 2052)               # rows of the output must be 16-byte aligned


def test_the_rotating_epilogue_needs_rounds_of_tiles_at_head_size_128():
    # head size 64: wherever the tcgen05 product runs
    assert gemm.rotating_epilogue_pays(17, 3072, 64) and gemm.rotating_epilogue_pays(2048, 3072, 64)
    # head size 128: from 2.4 rounds of 256-wide tiles over 148 SMs (356 tiles)
    assert not gemm.rotating_epilogue_pays(544, 5120, 128)           # 5 x 20 tiles: a 512-token portion of the 3B shape
    assert not gemm.rotating_epilogue_pays(2048, 5120, 128)          # 16 x 20 = 320
    assert gemm.rotating_epilogue_pays(2048, 6144, 128)              # 16 x 24 = 384
    assert gemm.rotating_epilogue_pays(4096, 5120, 128)
    # a head size the epilogue does not take
    assert not gemm.rotating_epilogue_pays(4096, 5120, 96)


def test_the_tcgen05_product_numbers_every_output_tile_once():
    """The kernel's own numbering of its output tiles (groups of row blocks, the row block changing fastest inside a
    group), called on the host: every tile of the grid has exactly one number, whatever the sizes, and consecutive
    numbers inside a group share their column block."""
    import pytest
    from dynalm_b200.kernels import ops
    if ops.CHECKED:
        pytest.skip("the checked build reads its record from the device after every call")
    import random
    rnd = random.Random(5)
    shapes = [(1, 1, 1), (5, 20, 16), (16, 112, 16), (64, 16, 9), (7, 3, 4), (33, 5, 16), (3, 7, 8)]
    shapes += [(rnd.randint(1, 70), rnd.randint(1, 40), rnd.randint(1, 20)) for _ in range(12)]
    for tiles_m, tiles_n, group_m in shapes:
        total = tiles_m * tiles_n
        seen = {}
        for tile in range(total):
            m, n = ops.gemm_tcgen05_tile_coords(tile, tiles_n, total, group_m)
            assert 0 <= m < tiles_m and 0 <= n < tiles_n, (tiles_m, tiles_n, group_m, tile, m, n)
            assert (m, n) not in seen, f"tiles {seen[(m, n)]} and {tile} are both ({m}, {n})"
            seen[(m, n)] = tile
        assert len(seen) == total
        rows = min(group_m, tiles_m)                          # the first group: numbers 0 .. rows - 1 are one column block
        first = [ops.gemm_tcgen05_tile_coords(t, tiles_n, total, group_m) for t in range(rows)]
        assert [m for m, _ in first] == list(range(rows)) and {n for _, n in first} == {0}
    with pytest.raises(Exception):
        ops.gemm_tcgen05_tile_coords(20, 4, 20, 2)           # past the last tile


def test_decode_attention_splits():
    # the 1B shape at 2,048 keys: powers of two (the splits of a row are one thread-block cluster), about one block per SM
    assert [attention.decode_splits(rows, 32, 8, 2048, sms=148) for rows in (1, 2, 4, 6, 8, 10)] == [8, 4, 4, 2, 2, 2]
    assert attention.decode_splits(64, 32, 8, 2048, sms=148) == 1
    # the same at 8,192 keys; more splits (merged by the second kernel) only from 32,768 keys on
    assert attention.decode_splits(1, 32, 8, 8192, sms=148) == 8
    assert attention.decode_splits(8, 32, 8, 8192, sms=148) == 2
    assert attention.decode_splits(1, 32, 8, 65536, sms=148) > 8
    # never less than 128 keys per split
    assert attention.decode_splits(1, 32, 8, 256, sms=148) == 2
    assert attention.decode_splits(1, 32, 8, 100, sms=148) == 1
    # the plain kernel (float32, large head sizes) has no cluster: as many splits as fill the GPU
    assert attention.decode_splits(8, 32, 8, 2048, tensor_cores=False, sms=148) == 3
    assert attention.decode_splits(1, 32, 8, 2048, tensor_cores=False, sms=148) == 16


def test_check_records_are_decoded():
    """Every code of the checked kernel build (csrc/check.cuh) has its sentence; 0 means nothing happened."""
    from dynalm_b200.kernels import ops
    assert ops.decode_check_record([0] * 8) == ""
    for code, words in ops.CHECK_CODES.items():
        text = ops.decode_check_record([code, -1, 0, 8, 3, 1, 0, 17])
        assert words in text and "-1 is not in [0, 8)" in text and "block 3,1,0, thread 17" in text
    assert "check code 99" in ops.decode_check_record([99, 1, 0, 1, 0, 0, 0, 0])
    src = open(os.path.join(os.path.dirname(ops.__file__), "..", "csrc", "check.cuh")).read()
    import re
    assert sorted(int(m) for m in re.findall(r"#define DL_CK_\w+ (\d+)", src)) == sorted(ops.CHECK_CODES)


def test_decode_units_deal_keys_evenly():
    """The plan of the split-KV decode attention: units of about equal size, never more than the grid holds, every row
    at least one part, short rows not cut below a tile per warp."""
    from dynalm_b200.kernels import attention as fast
    from dynalm_b200.kernels.attention import PART_CAP, DecodeUnits
    from dynalm_b200.engine.step import StepShape
    import numpy as np
    plan = DecodeUnits(chunks=8, tile_keys=32, window=0)
    few = plan.fill(np.zeros(plan.ints(0, 64), dtype=np.int32), StepShape([1] * 4, [0, 1, 2, 3], [99] * 4, [0, 1, 2, 3], 4))
    assert few == (0, 4)                                   # below a dozen rows the engine does not plan
    fast.PLANNED_MIN_ROWS, before = 1, fast.PLANNED_MIN_ROWS
    slots = plan.slots()
    assert plan.parts([2048] * 8) in ([5, 5, 5, 5, 5, 4, 4, 4],) and sum(plan.parts([2048] * 8)) * 8 <= slots
    assert plan.parts([2048]) == [16]                      # one row: as many parts as leave a tile per warp
    assert plan.parts([100]) == [1] and plan.parts([1]) == [1]
    assert plan.parts([2048] * 64) == [1] * 64             # more rows than a round of blocks: no cutting
    uneven = plan.parts([8000, 100, 100, 100])
    assert uneven[0] > 10 and uneven[1:] == [1, 1, 1]      # the long row gets the units
    assert max(plan.parts([100000] * 2)) <= PART_CAP
    rng = np.random.RandomState(0)
    for _ in range(200):
        rows = int(rng.randint(1, 65))
        counts = [int(n) for n in rng.randint(1, 9000, rows)]
        parts = plan.parts(counts)
        assert len(parts) == rows and min(parts) >= 1 and sum(parts) * 8 <= plan.unit_cap(rows)
        host = np.zeros(plan.ints(0, 64), dtype=np.int32)
        shape = StepShape([1] * rows, list(range(rows)), [n - 1 for n in counts], list(range(rows)), rows)
        units, got_rows = plan.fill(host, shape)
        assert got_rows == rows and units == sum(parts) * 8 == host[0]
        listed = host[4:4 + 4 * units].reshape(-1, 4)
        assert sorted(map(tuple, listed)) == sorted((r, c, p, parts[r]) for r in range(rows) for c in range(8) for p in range(parts[r]))
    windowed = DecodeUnits(chunks=2, tile_keys=16, window=64)
    assert windowed.parts([64, 64]) == windowed.parts([64, 64]) and windowed.fill(np.zeros(4000, dtype=np.int32),
        StepShape([1, 1, 5], [0, 1, 2], [9999, 10, 0], [0, 1, 2], 7))[1] == 2
    fast.PLANNED_MIN_ROWS = before


def test_query_tile_parts_deal_long_tiles(monkeypatch):
    """The plan of the tcgen05 prompt attention: tiles far longer than an even share of the step's work are cut into
    parts of at least 8 key tiles; short steps and steps with plenty of tiles are left whole; every entry names its
    part, the number of parts and the first record of its tile."""
    import numpy as np
    from dynalm_b200.engine.step import StepShape
    from dynalm_b200.kernels import attention as fast
    monkeypatch.setattr(fast, "sm_count", lambda: 148)
    plan = fast.QueryTileParts(n_heads=32, window=0)
    assert plan.key_tiles(0, 128) == 2 and plan.key_tiles(1920, 128) == 32 and plan.key_tiles(64, 1) == 2
    assert fast.QueryTileParts(8, 100).key_tiles(1000, 10) == 2              # a window: keys 901 .. 1009
    # one 2,048-token prompt: 16 tiles of 2 .. 32 key tiles: parts of fewer than 24 key tiles do not pay, all whole
    assert plan.deal([2 * (t + 1) for t in range(16)]) == [1] * 16
    # a 512-row portion at 32,768 keys: four tiles of about 510 key tiles, 128 blocks for 296 places: in four parts each
    assert plan.deal([506, 508, 510, 512]) == [4, 4, 4, 4]
    # the same at 8,192 keys (125 key tiles: parts of 31) and at 4,096 (62: two parts of 31); at 2,048 whole
    assert plan.deal([122, 124, 126, 128]) == [4, 4, 4, 4] and plan.deal([58, 60, 62, 64]) == [2, 2, 2, 2]
    assert plan.deal([26, 28, 30, 32]) == [1, 1, 1, 1]
    assert plan.deal([3, 4, 5]) == [1, 1, 1] and plan.deal([]) == []
    assert plan.deal([2 * (t + 1) for t in range(64)]) == [1] * 64            # an 8,192-token prompt: enough tiles
    assert sum(p for p in plan.deal([600] * 40) if p > 1) <= fast.PART_SLOTS   # no more parts than records
    host = np.zeros(plan.ints(2048, 8), dtype=np.int32)
    shape = StepShape([1, 1, 510], [0, 1, 2], [70, 9, 6000], [5, 6, 7], 512)   # two decode rows, then a portion at 6,000
    entries, records, cap = plan.fill(host, shape)
    assert cap == 2048 // 128 + 8 + fast.PART_SLOTS and records == 16 and entries == 4 * 4
    tiles = host[4:4 + 4 * entries].reshape(-1, 4)
    words = host[4 + 4 * cap:4 + 4 * cap + entries]
    assert set(tiles[:, 0]) == {7} and tiles[:, 1].min() == 2                  # the prompt's rows only
    seen = {}
    for (slot, row0, rows, pos0), w in zip(tiles.tolist(), words.tolist()):
        part, parts, record = w & 0xff, (w >> 8) & 0xff, w >> 16
        seen.setdefault((row0, rows, pos0), []).append((part, parts, record))
    assert len(seen) == 4
    for key, got in seen.items():
        parts = got[0][1]
        assert (parts == 0 and got == [(0, 0, 0)]) or (sorted(p for p, _, _ in got) == list(range(parts)) and
                                                       len({(n, r) for _, n, r in got}) == 1)
    firsts = sorted(got[0][2] for got in seen.values() if got[0][1] > 1)
    assert firsts == list(range(0, records, 4))                                # records of the split tiles do not overlap
