"""The entry point that allocates nothing, called through its exported C symbol.

Some users of the kernel library have no allocator to turn to: a C or Rust host, or a plugin inside
another server, whose device memory was divided up at start-up and which may not call cudaMalloc on
its token path (it stalls the whole device). For them `dl_paged_attention_decode_noalloc` keeps the
split-KV scratch inside the library. This test loads the built library with ctypes, calls that symbol
and the ordinary entry point (which is given scratch by the caller) on the same inputs, and wants the
same output within the tolerance of the other bfloat16 kernel tests; twice in a row, because the
built-in scratch keeps what the previous call left there. It also checks that a call too big for the
built-in scratch is refused, not run.

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
    g = torch.Generator(device="cpu").manual_seed(seed)
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 3
    perm = torch.randperm(pages, generator=g)
    table = torch.zeros(len(lens), max_blocks, dtype=torch.int32)
    nxt = 0
    for r, l in enumerate(lens):
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            nxt += 1
    kc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
    vc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
    q = torch.randn(rows, heads * hd, generator=g).to(torch.bfloat16)
    req = torch.arange(rows, dtype=torch.int32) % len(lens)
    pos = torch.tensor([lens[int(r)] - 1 for r in req], dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, table, pos, req)]


def test_no_alloc_entry_matches_the_ordinary_one():
    lib = _library()
    P, I, F = c_void_p, c_int, c_float
    noalloc = lib.dl_paged_attention_decode_noalloc
    noalloc.argtypes = [P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, F, I, I, P]
    noalloc.restype = c_int
    ordinary = lib.dl_paged_attention_decode_tc
    ordinary.argtypes = [P, I, P, P, P, I, P, P, P, I, P, I, I, I, I, I, F, I, I, P]
    ordinary.restype = c_int
    strerror = lib.dl_noalloc_strerror
    strerror.argtypes = [c_int]
    strerror.restype = ctypes.c_char_p

    heads, kvh, hd, page = 8, 2, 64, 16
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different inputs and split counts: the second finds the first one's
    # partial results in the shared scratch and must not be disturbed by them
    for seed, rows, lens, splits in ((1, 4, [700, 33, 260, 129], 5), (2, 3, [90, 513, 40], 3)):
        q, kc, vc, table, pos, req = _case(seed, rows, heads, kvh, hd, page, lens)
        scale = 1.0 / math.sqrt(hd)
        want = torch.zeros(rows, heads * hd, dtype=torch.bfloat16, device=DEV)
        scratch = torch.zeros(rows * heads * splits * (hd + 2), dtype=torch.float32, device=DEV)
        rc = ordinary(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0),
                      pos.data_ptr(), req.data_ptr(), want.data_ptr(), want.stride(0), scratch.data_ptr(), rows, heads,
                      kvh, hd, page, scale, 0, splits, stream)
        assert rc == 0, strerror(rc)
        got = torch.zeros_like(want)
        before = torch.cuda.memory_allocated()
        rc = noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0),
                     pos.data_ptr(), req.data_ptr(), got.data_ptr(), got.stride(0), rows, heads, kvh, hd, page, scale, 0,
                     splits, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2e-2, f"no-alloc entry differs from the ordinary one by {err}"
        assert got.float().abs().max().item() > 0

    # beyond the built-in scratch: refused with its own code, nothing launched, output untouched
    q, kc, vc, table, pos, req = _case(3, 4, heads, kvh, hd, page, [64, 64, 64, 64])
    out = torch.full((4, heads * hd), 7.0, dtype=torch.bfloat16, device=DEV)
    rc = noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(), table.stride(0), pos.data_ptr(),
                 req.data_ptr(), out.data_ptr(), out.stride(0), 40000, heads, kvh, hd, page, 0.125, 0, 8, stream)
    assert rc == 10002 and b"more scratch" in strerror(rc)
    torch.cuda.synchronize()
    assert (out == 7.0).all()
