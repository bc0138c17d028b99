"""The list of a layer's launches, issued again for the next layer by address (engine/launch_memo.py): which
arguments are exchanged, and when a list may not be reused. No GPU: the launches are stand-ins that note their
arguments."""

from dataclasses import dataclass

import torch

from dynalm_b200.engine import launch_memo
from dynalm_b200.engine.launch_memo import LayerLaunchMemo
from dynalm_b200.kernels import ops
from dynalm_b200.parts.block import ResidualStream


@dataclass(frozen=True)
class Spec:
    width: int


class Cache:
    def __init__(self, width):
        self.arrays = [torch.zeros(4, width), torch.zeros(4, width)]
        self.block_table = torch.zeros(2, 3, dtype=torch.int32)


class Block:
    """Stands for a block whose device work is three launches: one reads the weight from its third row on, one
    takes the cache arrays, one is a library product handed the weight itself."""

    replay_safe = True

    def __init__(self, width, log, dtype=torch.float32):
        self.spec = Spec(width)
        self.weight = torch.zeros(8, width, dtype=dtype)
        self.bias = torch.zeros(width)
        self.log = log
        self.scratch = None           # shared between layers: set by the test
        self.calls = 0                # times the block's own code ran

    def forward(self, stream, ctx, cache, owns_cache):
        self.calls += 1
        log = self.log

        def launch_a(*args):
            log.append(("a",) + args)
            return 0

        def launch_b(*args):
            log.append(("b",) + args)
            return 0

        def product(x, w, out):
            log.append(("mm", x.data_ptr(), w.data_ptr(), out.data_ptr()))
            return 0
        row = self.weight.stride(0) * self.weight.element_size()
        for f, args in ((launch_a, (self.weight.data_ptr() + 2 * row, self.scratch.data_ptr(), 7, 0.5)),
                        (launch_b, (cache.arrays[0].data_ptr(), cache.arrays[1].data_ptr(), cache.block_table.data_ptr(),
                                    self.bias.data_ptr(), stream.x.data_ptr())),
                        (product, (self.scratch, self.weight, self.scratch))):
            f(*args)
            if ops._recording is not None:
                ops._recording.append((f, args))
        stream.pending, stream.pending_scale = self.scratch, 1.0
        return stream


def run_layers(blocks, caches, scratch, monkeypatch=None):
    kinds, seen = [], {}
    for b in blocks:
        kinds.append(seen.setdefault((type(b), b.spec), len(seen)))
    memo = LayerLaunchMemo({}, kinds)
    stream = ResidualStream(torch.zeros(3, 8))
    for b in blocks:
        b.scratch = scratch
    for i, b in enumerate(blocks):
        stream = memo.run(i, b, stream, None, caches[i], True)
    return stream


def test_later_layers_are_issued_with_their_own_addresses():
    log, scratch = [], torch.zeros(16)
    blocks = [Block(8, log) for _ in range(4)]
    caches = [Cache(8) for _ in range(4)]
    before = launch_memo.REPLAYED_LAYERS
    stream = run_layers(blocks, caches, scratch)
    # layer 0 enters with nothing pending, layer 1 with the scratch pending: both run their own code; 2 and 3 do not
    assert [b.calls for b in blocks] == [1, 1, 0, 0]
    assert launch_memo.REPLAYED_LAYERS - before == 2
    assert stream.pending is scratch and stream.pending_scale == 1.0
    assert len(log) == 12
    for i, b in enumerate(blocks):
        a, bb, mm = log[3 * i:3 * i + 3]
        row = b.weight.stride(0) * b.weight.element_size()
        assert a == ("a", b.weight.data_ptr() + 2 * row, scratch.data_ptr(), 7, 0.5)        # offset kept, the rest as it was
        assert bb == ("b", caches[i].arrays[0].data_ptr(), caches[i].arrays[1].data_ptr(),
                      caches[i].block_table.data_ptr(), b.bias.data_ptr(), stream.x.data_ptr())
        assert mm == ("mm", scratch.data_ptr(), b.weight.data_ptr(), scratch.data_ptr())  # the tensor itself exchanged


def test_a_list_is_not_reused_across_kinds_layouts_or_unsafe_blocks():
    log, scratch = [], torch.zeros(16)
    # another spec, another dtype of the weight, and a block that does not say replay_safe: each runs its own code
    blocks = [Block(8, log), Block(8, log), Block(8, log), Block(16, log), Block(8, log, torch.float64), Block(8, log)]
    blocks[5].replay_safe = False
    caches = [Cache(b.spec.width) for b in blocks]
    run_layers(blocks, caches, scratch)
    assert [b.calls for b in blocks] == [1, 1, 0, 1, 1, 1]


def test_work_that_was_not_written_down_forbids_reuse():
    log, scratch = [], torch.zeros(16)

    class Unrecorded(Block):
        def forward(self, stream, ctx, cache, owns_cache):
            ops.note_unrecorded_work()
            return super().forward(stream, ctx, cache, owns_cache)
    blocks = [Unrecorded(8, log) for _ in range(4)]
    run_layers(blocks, [Cache(8) for _ in range(4)], scratch)
    assert [b.calls for b in blocks] == [1, 1, 1, 1]


def test_a_failed_launch_is_reported():
    import pytest
    from dynalm_b200.errors import EngineError
    log, scratch = [], torch.zeros(16)

    class Failing(Block):
        def forward(self, stream, ctx, cache, owns_cache):
            stream = super().forward(stream, ctx, cache, owns_cache)
            if self is blocks[1] and ops._recording is not None:
                ops._recording.append((lambda *a: 700, ()))
            return stream
    blocks = [Failing(8, log) for _ in range(3)]
    with pytest.raises(EngineError, match="CUDA error 700"):
        run_layers(blocks, [Cache(8) for _ in range(3)], scratch)
