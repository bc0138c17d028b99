"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library have no allocator to turn to: a C or Rust host, or a plugin inside
another server, whose device memory was divided up at start-up and which may not call cudaMalloc on
its token path (it stalls the whole device). For them `dl_paged_attention_decode_noalloc` keeps the
split-KV scratch inside the library. This test loads the built library with ctypes and calls that symbol
and the ordinary entry point (which is given scratch by the caller) on the same inputs.

The kernel touches scratch only when it does not merge a row's key splits inside a thread-block cluster, which it
does for 2, 4 and 8 splits (clusters of other sizes place badly on the GPU). The first cases are
of that kind, so the library's own array is what carries the partial results: the output must then be the
same bits as the ordinary entry point's at the same split count (it is the same kernel on the same
numbers; only the address of the scratch differs), and both must agree with a float64 attention written
out in the test. The calls come one after the other with different inputs, shapes and split counts, since
the array keeps what the previous call left there. A small call that merges in a cluster follows, and one
that is too big for the array and must be refused, not run.

The file name makes pytest collect it last, so a run that stops at the first failure has already run
everything else.
"""

import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _library():
    from dynalm_b200.kernels import lib
    return ctypes.CDLL(lib.compile_library("attention_decode"))


def _case(seed, rows, heads, kvh, hd, page, lens):
    """`rows` decode rows over len(lens) requests in scattered pages; also the keys and values of every request
    in order, for the float64 reference."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 3
    perm = torch.randperm(pages, generator=g)
    table = torch.zeros(len(lens), max_blocks, dtype=torch.int32)
    kc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
    keys, vals = [], []
    nxt = 0
    for r, l in enumerate(lens):
        mine = []
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            mine.append(int(perm[nxt]))
            nxt += 1
        keys.append(kc[mine].reshape(-1, kvh, hd)[:l].double())
        vals.append(vc[mine].reshape(-1, kvh, hd)[:l].double())
    q = torch.randn(rows, heads * hd, generator=g).to(torch.bfloat16)
    req = torch.arange(rows, dtype=torch.int32) % len(lens)
    pos = torch.tensor([lens[int(r)] - 1 for r in req], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, table, pos, req)], keys, vals


def _reference(q, keys, vals, req, heads, kvh, hd, scale):
    """softmax(scale q k^T) v in float64, row by row and head by head, every row over all keys of its request."""
    rows = q.shape[0]
    out = torch.zeros(rows, heads, hd, dtype=torch.float64)
    qd = q.cpu().double().view(rows, heads, hd)
    for i in range(rows):
        k, v = keys[int(req[i])], vals[int(req[i])]
        for h in range(heads):
            kh, vh = k[:, h // (heads // kvh)], v[:, h // (heads // kvh)]
            out[i, h] = torch.softmax(scale * (kh @ qd[i, h]), 0) @ vh
    return out.view(rows, heads * hd)


def test_no_alloc_entry_matches_the_ordinary_one():
    lib = _library()
    P, I, F = c_void_p, c_int, c_float
    noalloc = lib.dl_paged_attention_decode_noalloc
    noalloc.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P]
    noalloc.restype = c_int
    ordinary = lib.dl_paged_attention_decode_tc
    ordinary.argtypes = [P, I, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, P, ctypes.c_longlong, P]
    ordinary.restype = c_int
    strerror = lib.dl_noalloc_strerror
    strerror.argtypes = [c_int]
    strerror.restype = ctypes.c_char_p

    heads, kvh, page = 8, 2, 16
    stream = torch.cuda.current_stream().cuda_stream
    if hasattr(lib, "dl_check_limits"):
        # a checked build of the library (csrc/check.cuh) compares page ids with the ranges that its last user set;
        # this test calls the kernels directly and sets none
        lib.dl_check_limits.argtypes = [I, I, I, I, P]
        assert lib.dl_check_limits(0, 0, 0, 0, stream) == 0
    many = [97, 33, 260, 129, 1, 700, 64, 65, 511, 48, 300, 17, 222, 16, 401, 130, 75, 999, 250, 31]
    cases = (
        # (seed, head size, rows, tokens each request holds, key splits, does the kernel merge through scratch?)
        (1, 64, 20, many, 3, True),                       # three splits: no cluster of that size
        (2, 64, 3, [1600, 2100, 1537], 12, True),         # more splits than a cluster can hold
        (3, 128, 24, many[:12], 5, True),                 # other shapes over the records the calls before left
        (4, 64, 20, many[::-1], 6, True),
        (6, 64, 20, many[::-1], 2, False),                # two splits: a cluster of two, however many rows
        (5, 64, 4, [700, 33, 260, 129], 4, False),        # four splits: merged inside a cluster
    )
    for seed, hd, rows, lens, splits, through_scratch in cases:
        assert through_scratch == (splits > 8 or splits & (splits - 1) != 0)
        (q, kc, vc, table, pos, req), keys, vals = _case(seed, rows, heads, kvh, hd, page, lens)
        scale = 1.0 / math.sqrt(hd)
        want = torch.zeros(rows, heads * hd, dtype=torch.bfloat16, device=DEV)
        scratch = torch.zeros(rows * heads * splits * (hd + 2), dtype=torch.float32, device=DEV)
        rc = ordinary(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0),
                      pos.data_ptr(), req.data_ptr(), want.data_ptr(), want.stride(0), scratch.data_ptr(), rows, heads,
                      kvh, hd, page, scale, 0, splits, None, 0, stream)
        assert rc == 0, strerror(rc)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        if through_scratch:
            assert scratch.abs().sum().item() > 0, "the ordinary call was expected to leave partial results in its scratch"
        before = torch.cuda.memory_allocated()
        rc = noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0),
                     pos.data_ptr(), req.data_ptr(), got.data_ptr(), got.stride(0), rows, heads, kvh, hd, page, scale, 0,
                     splits, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(got, want), (f"case {seed}: the no-alloc entry differs from the ordinary one by "
                                        f"{(got.float() - want.float()).abs().max().item()}")
        ref = _reference(q, keys, vals, req.cpu(), heads, kvh, hd, scale)
        for name, t in (("no-alloc", got), ("ordinary", want)):
            err = (t.cpu().double() - ref).abs().max().item()
            assert err <= 2.5e-2, f"case {seed}: the {name} entry is {err} away from the float64 attention"

    # beyond the built-in scratch: refused with its own code, nothing launched, output untouched
    (q, kc, vc, table, pos, req), _, _ = _case(6, 4, heads, kvh, 64, page, [64, 64, 64, 64])
    out = torch.full((4, heads * 64), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0), pos.data_ptr(),
                 req.data_ptr(), out.data_ptr(), out.stride(0), 40000, heads, kvh, 64, page, 0.125, 0, 8, stream)
    assert rc == 10002 and b"more scratch" in strerror(rc)
    torch.cuda.synchronize()
    assert (out == 7.0).all()
