"""The checked build of the kernels (DYNALM_CHECK=1, csrc/check.cuh) catches an index out of range, says which, does
not make the access and leaves the device usable. Run in a child process, since the switch is read when the package
is imported.

The wrong indices are chosen so that even an unchecked kernel would stay inside memory that the test owns: the cache
arrays handed to the kernels are the middle of a larger allocation, and the wrong page ids (-1 and one past the end)
point into its margins."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import torch
from dynalm_b200.errors import EngineError
from dynalm_b200.kernels import ops
assert ops.CHECKED
dev = "cuda:0"
heads, kvh, hd, page = 4, 2, 64, 16
pages = 8
big_k = torch.randn(pages + 2, page, kvh, hd, device=dev).to(torch.bfloat16)
big_v = torch.randn(pages + 2, page, kvh, hd, device=dev).to(torch.bfloat16)
kc, vc = big_k[1:pages + 1], big_v[1:pages + 1]           # pages -1 and `pages` lie in the margins
table = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=torch.int32, device=dev)
q = torch.randn(2, heads * hd, device=dev).to(torch.bfloat16)
out = torch.zeros_like(q)
pos = torch.tensor([40, 63], dtype=torch.int32, device=dev)
req = torch.tensor([0, 1], dtype=torch.int32, device=dev)
scratch = torch.zeros(4096, device=dev)

def decode():
    ops.paged_attention_decode(q, kc, vc, table, pos, req, out, scratch, heads, kvh, hd, page, 0.125, 0, 1, tensor_cores=True)

def generic():
    ops.paged_attention_generic(q, kc, vc, table, pos, req, out, heads, kvh, hd, page, 0.125)

def expect(f, words):
    try:
        f()
    except EngineError as e:
        assert all(w in str(e) for w in words), str(e)
        return
    raise AssertionError("no error for " + " ".join(words))

decode(); generic()                                   # all in range: nothing is reported
good = out.clone()
table[1, 2] = -1                                      # a page that a window has given back
expect(decode, ["a page id outside the pool", "-1 is not in [0, 8)"])
expect(generic, ["a page id outside the pool", "-1 is not in [0, 8)"])
table[1, 2] = pages                                   # one past the pool
expect(decode, ["a page id outside the pool", "8 is not in [0, 8)"])
table[1, 2] = 6
req[1] = 2                                            # a request the table has no row for
expect(decode, ["a request index outside the block table", "2 is not in [0, 2)"])
req[1] = 1
pos[1] = 64                                           # a position past the table's row
expect(generic, ["outside the request's row of the block table", "4 is not in [0, 4)"])
pos[1] = 63
# the record was cleared when it was read, the device is usable and the results are what they were
decode()
assert torch.equal(out, good) or (out.float() - good.float()).abs().max().item() < 2e-2
# stores: a key/value write to a page outside the pool is skipped, the cache keeps its contents
qkv = torch.randn(2, (heads + 2 * kvh) * hd, device=dev).to(torch.bfloat16)
inv = torch.ones(hd // 2, device=dev)
before_k = big_k.clone()
table[0, 2] = pages
expect(lambda: ops.rope_cache_write(qkv, pos, req, table, kc, vc, inv, hd, 1.0, heads, kvh, hd, page), ["a page id outside the pool"])
changed = (big_k != before_k).flatten(1).any(1).nonzero().flatten().tolist()
assert changed == [1 + 7], changed                    # only request 1's page (position 63 -> block 3 -> page 7) was written
# token ids and gathered rows
tab = torch.randn(10, 32, device=dev)
x = torch.zeros(3, 32, device=dev)
ids = torch.tensor([1, 10, 2], dtype=torch.int32, device=dev)
expect(lambda: ops.embed(tab, ids, x), ["a token id outside the vocabulary", "10 is not in [0, 10)"])
rows = torch.tensor([0, 3], dtype=torch.int32, device=dev)
y = torch.zeros(2, 32, device=dev)
expect(lambda: ops.rmsnorm(x, torch.ones(32, device=dev), 1e-5, y, rows=rows), ["a gathered row outside the rows of the step", "3 is not in [0, 3)"])
# the prompt attention's part words: a tile whose parts name records beyond the scratch is run whole instead, and said
table[0, 2], table[1, 2] = 2, 6
qp = torch.randn(64, heads * hd, device=dev).to(torch.bfloat16)
outp = torch.zeros_like(qp)
tiles = torch.tensor([[0, 0, 64, 0], [0, 0, 64, 0]], dtype=torch.int32, device=dev)
words = torch.tensor([0 | 2 << 8 | 3 << 16, 1 | 2 << 8 | 3 << 16], dtype=torch.int32, device=dev)       # records 3 and 4 of 4
partial = torch.zeros(4 * heads * (hd + 2) * 128, device=dev)
counters = torch.zeros(4 * heads, dtype=torch.int32, device=dev)
expect(lambda: ops.paged_attention_prefill_tcgen05(qp, kc, vc, table, tiles, 2, outp, heads, kvh, hd, page, 0.125,
                                                    unit_parts=words, partial=partial, counters=counters),
       ["a part of a query tile", "5 is not in [0, 5)"])
assert float(partial.abs().sum()) == 0.0 and int(counters.abs().sum()) == 0        # nothing was written beyond (or into) the scratch
torch.cuda.synchronize()
print("checked build ok")
'''


def test_checked_build_reports_and_skips():
    env = dict(os.environ, DYNALM_CHECK="1", PYTHONPATH=ROOT)
    proc = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=900)
    assert proc.returncode == 0 and "checked build ok" in proc.stdout, proc.stdout[-2000:] + proc.stderr[-4000:]
