"""Each kernel alone against a plain PyTorch fp32 reference of the same op, at sizes that are not
the engine's: widths and vocabularies that are no power of two, head sizes in steps of 16, odd
numbers of heads and groups, windows, pages entered in the middle."""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 2e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from dynalm_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab", [(80, 499), (2048, 1000), (24, 7)])
def test_embed(ops, dtype, width, vocab):
    g = torch.Generator(device="cpu").manual_seed(1)
    table = torch.randn(vocab, width, generator=g).to(DEV, dtype)
    ids = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(37, width, dtype=torch.float32, device=DEV)
    ops.embed(table, ids, out, 3.0)
    ref = table.float()[ids.long()] * 3.0
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 1000, 2048, 5120])
def test_rmsnorm_with_residual_and_rows(ops, dtype, width):
    g = torch.Generator(device="cpu").manual_seed(2)
    n = 19
    x = (torch.randn(n, width, generator=g) * 3).to(DEV)
    delta = torch.randn(n, width, generator=g).to(DEV, dtype)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    eps = 3e-5

    def ref_norm(v):
        v = v.double()
        return (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * w.double()).float()

    # plain
    out = torch.empty(n, width, dtype=dtype, device=DEV)
    ops.rmsnorm(x.clone(), w, eps, out)
    assert (out.float() - ref_norm(x)).abs().max() <= tol(dtype, 4)
    # fused residual add, written back
    x2 = x.clone()
    ops.rmsnorm(x2, w, eps, out, delta=delta, delta_scale=0.5)
    summed = x + 0.5 * delta.float()
    assert (x2 - summed).abs().max() <= 1e-6
    assert (out.float() - ref_norm(summed)).abs().max() <= tol(dtype, 4)
    # gathered rows: nothing written back
    rows = torch.tensor([18, 0, 7], dtype=torch.int32, device=DEV)
    x3 = x.clone()
    out3 = torch.empty(3, width, dtype=dtype, device=DEV)
    ops.rmsnorm(x3, w, eps, out3, delta=delta, delta_scale=0.5, rows=rows)
    assert torch.equal(x3, x)
    assert (out3.float() - ref_norm(summed[rows.long()])).abs().max() <= tol(dtype, 4)
    # pending add alone
    x4 = x.clone()
    ops.residual_add(x4, delta, 0.5)
    assert (x4 - summed).abs().max() <= 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    g = torch.Generator(device="cpu").manual_seed(3)
    gu = (torch.randn(13, 2 * 112, generator=g) * 4).to(DEV, dtype)
    out = torch.empty(13, 112, dtype=dtype, device=DEV)
    ops.silu_mul(gu, out)
    a, b = gu.float()[:, :112], gu.float()[:, 112:]
    ref = a * torch.sigmoid(a) * b
    assert (out.float() - ref).abs().max() <= tol(dtype, ref.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 499, 80), (37, 130, 200), (64, 64, 16), (200, 96, 1000), (5, 3, 7)])
def test_gemm_simt(ops, dtype, M, N, K):
    g = torch.Generator(device="cpu").manual_seed(4)
    x = torch.randn(M, K, generator=g).to(DEV, dtype)
    w = torch.randn(N, K, generator=g).to(DEV, dtype)
    bias = torch.randn(N, generator=g).to(DEV)
    ref = (x.double() @ w.double().T + bias.double()) * 0.25
    for out_dtype in ({torch.float32} | {dtype}):
        out = torch.empty(M, N, dtype=out_dtype, device=DEV)
        ops.gemm_simt(x, w, out, bias, 0.25)
        scale = ref.abs().max().item()
        assert (out.double() - ref).abs().max() <= (1e-5 if out_dtype == torch.float32 else 1e-2) * scale
    # a row's result does not depend on how many rows share the call
    if M > 1:
        one = torch.empty(1, N, dtype=torch.float32, device=DEV)
        full = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops.gemm_simt(x, w, full)
        ops.gemm_simt(x[M - 1:M], w, one)
        assert torch.equal(one[0], full[M - 1])


def _rope_ref(x, pos, inv_freq, rot, pos_scale):
    """x [n, heads, hd] fp64; half-split rotation of the first `rot` dims."""
    half = rot // 2
    theta = (pos.float() * pos_scale)[:, None] * inv_freq[None, :]          # fp32 product, as the kernel
    c, s = torch.cos(theta.double())[:, None, :], torch.sin(theta.double())[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:rot]
    out[..., :half] = a * c - b * s
    out[..., half:rot] = a * s + b * c
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,rot,page", [(5, 1, 48, 24, 16), (6, 2, 32, 32, 16), (3, 3, 80, 80, 32),
                                                     (8, 2, 128, 128, 16)])
def test_rope_cache_write(ops, dtype, heads, kvh, hd, rot, page):
    g = torch.Generator(device="cpu").manual_seed(5)
    n_req, max_blocks, pages = 3, 8, 40
    # three requests with rows at scattered positions; pages handed out in a shuffled order
    perm = torch.randperm(pages, generator=g)[: n_req * max_blocks].reshape(n_req, max_blocks).to(torch.int32)
    req = torch.tensor([0, 0, 0, 1, 2, 2, 1, 0], dtype=torch.int32)
    pos = torch.tensor([14, 15, 16, 0, 100, 101, 47, 127 if page * max_blocks > 127 else 17], dtype=torch.int32)
    n = len(req)
    width = (heads + 2 * kvh) * hd
    qkv = torch.randn(n, width, generator=g).to(DEV, dtype)
    inv = (10000.0 ** (-torch.arange(rot // 2).float() * 2 / rot)).to(DEV)
    kc = torch.zeros(pages, page, kvh, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    before = qkv.clone()
    ops.rope_cache_write(qkv, pos.to(DEV), req.to(DEV), perm.to(DEV), kc, vc, inv, rot, 0.5, heads, kvh, hd, page)
    src = before.double().cpu()
    q = src[:, :heads * hd].reshape(n, heads, hd)
    k = src[:, heads * hd:(heads + kvh) * hd].reshape(n, kvh, hd)
    v = src[:, (heads + kvh) * hd:].reshape(n, kvh, hd)
    q_ref = _rope_ref(q, pos, inv.cpu(), rot, 0.5)
    k_ref = _rope_ref(k, pos, inv.cpu(), rot, 0.5)
    t = tol(dtype, 4)
    assert (qkv[:, :heads * hd].double().cpu().reshape(n, heads, hd) - q_ref).abs().max() <= t
    for i in range(n):
        p = perm[req[i], pos[i] // page].item()
        s = pos[i].item() % page
        assert (kc[p, s].double().cpu() - k_ref[i]).abs().max() <= t, f"key of row {i}"
        assert torch.equal(vc[p, s].cpu(), before[i, (heads + kvh) * hd:].reshape(kvh, hd).cpu()), f"value of row {i}"
    # nothing else was touched
    written = torch.zeros(pages, page, dtype=torch.bool)
    for i in range(n):
        written[perm[req[i], pos[i] // page], pos[i] % page] = True
    assert kc.cpu()[~written].abs().max() == 0 and vc.cpu()[~written].abs().max() == 0


def _attention_ref(q, keys, vals, scale, window):
    """One row: q [heads, hd], keys/vals [t, kvh, hd] (positions 0..t-1, the row is at t-1)."""
    heads, hd = q.shape
    kvh = keys.shape[1]
    t = keys.shape[0]
    lo = max(0, t - window) if window > 0 else 0
    out = torch.zeros(heads, hd, dtype=torch.float64)
    for h in range(heads):
        kh = keys[lo:, h // (heads // kvh)]
        vh = vals[lo:, h // (heads // kvh)]
        s = scale * (kh @ q[h])
        p = torch.softmax(s, 0)
        out[h] = p @ vh
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kvh,hd,page,window", [(4, 2, 16, 16, 0), (6, 2, 32, 16, 0), (5, 1, 48, 16, 0),
                                                        (3, 3, 80, 32, 0), (8, 2, 128, 16, 40), (2, 1, 256, 16, 0),
                                                        (4, 4, 64, 16, 7)])
def test_paged_attention_generic(ops, dtype, heads, kvh, hd, page, window):
    """Three requests in scattered pages (60 / 700 / 130 tokens); a batch that mixes a decode row, a
    portion that starts in the middle of a page, a short run and another decode row. One far key is
    made to stand out so that a kernel that skips or repeats a page cannot pass."""
    g = torch.Generator(device="cpu").manual_seed(6)
    lens = [60, 700, 130]
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 5
    perm = torch.randperm(pages, generator=g)
    table = torch.full((3, max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(pages, page, kvh, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    keys, vals = [], []
    nxt = 0
    for r, l in enumerate(lens):
        k = torch.randn(l, kvh, hd, generator=g).to(dtype)
        v = torch.randn(l, kvh, hd, generator=g).to(dtype)
        k[3] *= 4.0                               # a far key with a large score for matching queries
        keys.append(k)
        vals.append(v)
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            nxt += 1
            n = min(page, l - b * page)
            kc[table[r, b], :n] = k[b * page:b * page + n]
            vc[table[r, b], :n] = v[b * page:b * page + n]
    # rows: (request, position)
    rows = [(0, 59)] + [(1, p) for p in range(700 - 210, 700)] + [(2, p) for p in range(100, 105)] + [(2, 129)]
    # one row of request 1 is taken out and put last, as a second decode-like row would be
    req = torch.tensor([r for r, _ in rows], dtype=torch.int32)
    pos = torch.tensor([p for _, p in rows], dtype=torch.int32)
    n = len(rows)
    q = torch.randn(n, heads, hd, generator=g).to(dtype)
    for i, (r, p) in enumerate(rows):
        if i % 3 == 0:
            q[i, :, :] = (keys[r][3, 0].float() * 0.5).to(dtype)     # points at the far key
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(n, heads * hd, dtype=dtype, device=DEV)
    ops.paged_attention_generic(q.reshape(n, heads * hd).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV),
                                pos.to(DEV), req.to(DEV), out, heads, kvh, hd, page, scale, window)
    got = out.double().cpu().reshape(n, heads, hd)
    for i, (r, p) in enumerate(rows):
        ref = _attention_ref(q[i].double(), keys[r][:p + 1].double(), vals[r][:p + 1].double(), scale, window)
        err = (got[i] - ref).abs().max().item()
        assert err <= tol(dtype, 2), f"row {i} (request {r}, position {p}): {err}"


def test_argmax_ties_and_sizes(ops):
    g = torch.Generator(device="cpu").manual_seed(7)
    # 50,001: rows that do not start on 16 bytes and a last slice that is no multiple of 4 (the scan's scalar ends)
    for vocab in (7, 499, 50001, 50004, 128256):
        logits = torch.randn(5, vocab, generator=g)
        logits[1, 3] = logits[1].max() + 1
        logits[1, min(6, vocab - 1)] = logits[1, 3]              # a tie: the lowest id wins
        logits[2, vocab - 1] = 50.0
        logits[3, 0] = 50.0
        if vocab > 45000:                                        # a tie between two slices of the scan
            logits[4, 10001] = 60.0
            logits[4, 40002] = 60.0
            logits[2, vocab - 3] = 50.0                          # and one inside the last slice's ragged end
        d = logits.to(DEV)
        out = torch.empty(5, dtype=torch.int32, device=DEV)
        ops.argmax(d, out)
        ref = [int(np.flatnonzero(row == row.max())[0]) for row in logits.numpy()]
        assert out.cpu().tolist() == ref


def test_sample_temperature_matches_walk(ops):
    from plain_llama import sample_temperature
    g = torch.Generator(device="cpu").manual_seed(8)
    # one block a row up to 16,384 ids, then clusters of 2, 4 and 8 blocks; 50,001: rows that do not start on 16 bytes
    for vocab, rows in ((11, 64), (499, 64), (5000, 64), (20000, 16), (50001, 16), (128256, 16), (300000, 8)):
        logits = torch.randn(rows, vocab, generator=g) * 3
        temps = torch.full((rows,), 0.8)
        u = torch.rand(rows, generator=g, dtype=torch.float64)
        u[0] = 0.0                                              # the first id with any mass
        u[1] = 0.9999999                                        # the far end of the walk
        if vocab > 1000:
            logits[0, :700] = -float("inf")                     # ... which lies past the first threads' runs
            logits[1, vocab - 900:] = -float("inf")             # ... and the last mass before the last threads' runs
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        ops.sample_temperature(logits.to(DEV), temps.to(DEV), u.to(DEV), out)
        got = out.cpu().tolist()
        agree = 0
        for r in range(rows):
            ref = sample_temperature(logits[r].numpy(), 0.8, float(u[r]))
            # a draw that lands within rounding of a boundary may fall to the neighbour
            agree += got[r] == ref
            assert abs(got[r] - ref) <= 1, f"vocab {vocab} row {r}: {got[r]} vs {ref}"
        assert agree >= rows - 2
        if vocab > 1000:
            assert got[0] == 700


def test_sample_temperature_frequencies(ops):
    """20 000 draws: empirical frequencies within 0.015 of softmax(l / T)
    (the reference's own check, dynalm/tests/test_engine.cpp:507-680)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]])
    T = 0.7
    n = 20000
    g = torch.Generator(device="cpu").manual_seed(9)
    u = torch.rand(n, generator=g, dtype=torch.float64).to(DEV)
    big = logits.repeat(n, 1).to(DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample_temperature(big, torch.full((n,), T, device=DEV), u, out)
    freq = torch.bincount(out.cpu().long(), minlength=5).double() / n
    p = torch.softmax(logits[0].double() / T, 0)
    assert (freq - p).abs().max() < 0.015


def test_apply_penalties_matches_the_host(ops):
    """The penalties kernel against the host's (sampler.cpp:96-116): the same float32 bits on the rows it names, the
    other rows untouched."""
    from dynalm_b200.sampling import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    g = torch.Generator(device="cpu").manual_seed(12)
    vocab = 5003
    logits = torch.randn(6, vocab, generator=g) * 4
    contexts = {1: [7, 7, 7, 12, 5002, 0, 12], 4: list(range(40, 140)) + [41] * 5, 5: []}
    params = {1: SamplingParams(temperature=0.7, repetition_penalty=1.3, frequency_penalty=0.2, presence_penalty=-0.4),
              4: SamplingParams(temperature=0.7, repetition_penalty=0.8, penalty_last_n=-1),
              5: SamplingParams(temperature=0.7, presence_penalty=1.0)}
    def triples_of(contexts, unseen):
        rows, triples, pp, first = [], [], [], [0]
        for j, r in enumerate(sorted(contexts)):
            s = Sampler(params[r])
            ids, counts = s.penalty_counts(contexts[r], vocab, unseen=unseen.get(r, 0))
            rows.append(r)
            pp.append((params[r].repetition_penalty, params[r].frequency_penalty, params[r].presence_penalty))
            triples += [(j, int(i), int(c)) for i, c in zip(ids, counts)]
            first.append(len(triples))
        return (torch.tensor(rows, dtype=torch.int32, device=DEV),
                torch.tensor(triples or [(0, 0, 0)], dtype=torch.int32, device=DEV), len(triples),
                torch.tensor(pp, dtype=torch.float32, device=DEV), torch.tensor(first, dtype=torch.int32, device=DEV))

    want = logits.clone().numpy()
    for r in contexts:
        Sampler(params[r]).apply_penalties(want[r], contexts[r])
    d = logits.to(DEV)
    rows, triples, n, pp, first = triples_of(contexts, {})
    ops.apply_penalties(d, rows, triples, n, pp, first)
    assert np.array_equal(d.cpu().numpy(), want)
    assert not np.array_equal(want[1], logits[1].numpy()) and np.array_equal(want[0], logits[0].numpy())
    # The last token of each context known to the device only (a step in flight chose it): a token that is in
    # the context already (7 in row 1), one that is new to it (41 leaves row 4's list when it is taken away ... it
    # does not: it occurs six times), and one that is the whole context (row 5).
    contexts2 = {1: contexts[1] + [7], 4: contexts[4] + [4000], 5: [321]}
    want2 = logits.clone().numpy()
    for r in contexts2:
        Sampler(params[r]).apply_penalties(want2[r], contexts2[r])
    d2 = logits.to(DEV)
    rows, triples, n, pp, first = triples_of({r: c[:-1] for r, c in contexts2.items()}, {r: 1 for r in contexts2})
    chosen = torch.tensor([0, 4000, 7, 0, 321], dtype=torch.int32, device=DEV)
    pending = torch.tensor([2, 1, 4], dtype=torch.int32, device=DEV)
    ops.apply_penalties(d2, rows, triples, n, pp, first, chosen=chosen, pending=pending)
    assert np.array_equal(d2.cpu().numpy(), want2)
    # with a window, the token in flight takes the place of the oldest one
    windowed = SamplingParams(temperature=0.7, repetition_penalty=1.2, frequency_penalty=0.3, penalty_last_n=4)
    params[2] = windowed
    ctx = [9, 8, 7, 6, 5]
    want3 = logits.clone().numpy()
    Sampler(windowed).apply_penalties(want3[2], ctx)
    d3 = logits.to(DEV)
    rows, triples, n, pp, first = triples_of({2: ctx[:-1]}, {2: 1})
    ops.apply_penalties(d3, rows, triples, n, pp, first, chosen=torch.tensor([5], dtype=torch.int32, device=DEV),
                        pending=torch.tensor([0], dtype=torch.int32, device=DEV))
    assert np.array_equal(d3.cpu().numpy(), want3)
    assert want3[2, 9] == logits[2, 9] and want3[2, 8] != logits[2, 8]


def _peaked_logits(rows, vocab, g, spread):
    """Logits like a model's: a few ids stand out, the rest fall away (so that a nucleus is tens of ids, not most of
    the vocabulary), with some exactly equal values among the largest."""
    logits = torch.randn(rows, vocab, generator=g) * spread - 12.0
    top = torch.randint(0, vocab, (rows, 12), generator=g)
    for r in range(rows):
        logits[r, top[r]] += torch.linspace(9.0, 4.0, 12)
        logits[r, top[r, 5]] = logits[r, top[r, 4]]              # a tie inside every top-k of 5 or more
    return logits


@pytest.mark.parametrize("vocab", [300, 5003, 128256])
def test_sample_filtered_matches_the_host_pipeline(ops, vocab):
    """Top-k, min-p and top-p on the device against the host's pipeline (sampler.cpp:120-220) with the same uniform
    numbers: the same id, except where the draw lands within rounding of a boundary between two candidates (then
    the neighbour in the pipeline's order, which for the test must at least be one of the row's candidates)."""
    from dynalm_b200.sampling import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    g = torch.Generator(device="cpu").manual_seed(vocab)
    combos = [dict(top_k=40), dict(top_k=5), dict(top_k=1000), dict(top_p=0.9), dict(top_p=0.5), dict(top_k=50, top_p=0.8),
              dict(top_k=40, min_p=0.05), dict(top_p=0.95, min_p=0.02), dict(top_k=20, top_p=0.9, min_p=0.1),
              dict(top_k=vocab + 5, top_p=0.7), dict(top_k=2), dict(top_p=0.999)]
    rows = 4 * len(combos)
    logits = _peaked_logits(rows, vocab, g, 1.0)
    logits[3, :17] = -float("inf")                           # masked ids take no part
    u = torch.rand(rows, generator=g, dtype=torch.float64)
    u[0], u[1] = 0.0, 1.0 - 2.0 ** -40
    temps = [0.7, 1.0, 1.6, 0.3]
    params = [SamplingParams(temperature=temps[r % 4], **combos[r // 4]) for r in range(rows)]
    samplers = [Sampler(p) for p in params]
    dparams = torch.tensor([[p.temperature, s.cut_offset, p.top_p, float(u[r])] for r, (p, s) in enumerate(zip(params, samplers))],
                           dtype=torch.float64)
    order = torch.randperm(rows, generator=g)                # selections in another order than the rows
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    ops.sample_filtered(logits.to(DEV), order.to(torch.int32).to(DEV), rows, dparams[order].to(DEV),
                        torch.tensor([params[int(r)].top_k for r in order], dtype=torch.int32, device=DEV), out)
    got = out.cpu().tolist()
    same = host = 0
    for r in range(rows):
        ref = samplers[r].sample_host(logits[r].numpy().copy(), [], u=float(u[r]))
        if got[r] == ops.SAMPLE_FILTERED_HOST:
            # allowed where no filter is in effect (top-k of the vocabulary or more, no top-p), or where top-p alone
            # keeps more ids than the kernel holds
            p = params[r]
            l = logits[r].double()
            probs = torch.sort(torch.exp((l - l.max()) / p.temperature), descending=True).values
            nucleus = int((torch.cumsum(probs, 0) < p.top_p * probs.sum()).sum()) + 1
            assert (p.top_k >= vocab and p.top_p >= 1.0) or (not 0 < p.top_k < vocab and nucleus > 900), \
                f"vocab {vocab} row {r} {combos[r // 4]}: left to the host with a nucleus of {nucleus}"
            host += 1
            continue
        same += got[r] == ref
        assert got[r] == ref or abs(float(logits[r, got[r]]) - float(logits[r, ref])) < 0.2, \
            f"vocab {vocab} row {r} {combos[r // 4]}: {got[r]} vs {ref}"
    assert host <= rows // 3 and same >= rows - host - 1, (same, host)


def test_sample_filtered_with_a_wide_nucleus(ops):
    """Nearly flat logits: top-p keeps most of 128,256 ids, far more than the kernel can hold as candidates; it finds
    the end of the nucleus and the drawn id by narrowing the row down to one bin at a time. Against the host's
    pipeline with the same uniform numbers. Top-k of more than the kernel holds is left to the host."""
    from dynalm_b200.sampling import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    g = torch.Generator(device="cpu").manual_seed(3)
    vocab, rows = 128256, 9
    logits = torch.randn(rows, vocab, generator=g) * 0.1
    logits[2, 1000:1200] = logits[2, 999]                    # two hundred equal logits in the middle of a nucleus
    logits[5] = 0.25                                         # a row of equal logits: their order is that of the ids
    u = torch.rand(rows, generator=g, dtype=torch.float64)
    params = [SamplingParams(temperature=0.8, top_p=[0.9, 0.5, 0.99][r % 3], min_p=0.5 if r == 7 else 0.0,
                             top_k=5000 if r == 8 else 0) for r in range(rows)]
    samplers = [Sampler(p) for p in params]
    dparams = torch.tensor([[p.temperature, s.cut_offset, p.top_p, float(u[r])] for r, (p, s) in enumerate(zip(params, samplers))],
                           dtype=torch.float64, device=DEV)
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    ops.sample_filtered(logits.to(DEV), torch.arange(rows, dtype=torch.int32, device=DEV), rows, dparams,
                        torch.tensor([p.top_k for p in params], dtype=torch.int32, device=DEV), out)
    got = out.cpu().tolist()
    assert got[8] == ops.SAMPLE_FILTERED_HOST
    answered = [r for r in range(rows) if r != 8]
    refs = {r: samplers[r].sample_host(logits[r].numpy().copy(), [], u=float(u[r])) for r in answered}
    assert sum(got[r] == refs[r] for r in answered) >= len(answered) - 1, (got, refs)
    for r in answered:
        assert got[r] == refs[r] or abs(float(logits[r, got[r]]) - float(logits[r, refs[r]])) < 1e-3, (r, got[r], refs[r])


def test_sample_filtered_with_more_equal_logits_than_candidates(ops):
    """Thousands of ids share the logit on which top-k or the nucleus ends: among equal logits the order is that of
    the ids, and the kernel follows it without sorting them. Against the host's pipeline."""
    from dynalm_b200.sampling import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    g = torch.Generator(device="cpu").manual_seed(31)
    vocab, rows = 50000, 8
    logits = torch.randn(rows, vocab, generator=g) - 6.0
    for r in range(rows):
        logits[r, 100 * r:100 * r + 7] = torch.linspace(3.0, 2.0, 7)          # a few ids above the plateau
        logits[r, 20000 + r:20000 + r + 3000] = 1.5                           # the plateau: 3,000 equal logits
    u = torch.tensor([0.0, 0.3, 0.6, 0.9, 0.95, 0.5, 0.7, 0.999], dtype=torch.float64)
    params = [SamplingParams(temperature=1.0, top_k=[50, 500, 1000, 8][r % 4]) if r < 4 else
              SamplingParams(temperature=1.0, top_p=[0.5, 0.9, 0.99, 0.7][r % 4]) for r in range(rows)]
    samplers = [Sampler(p) for p in params]
    dparams = torch.tensor([[p.temperature, s.cut_offset, p.top_p, float(u[r])] for r, (p, s) in enumerate(zip(params, samplers))],
                           dtype=torch.float64, device=DEV)
    out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    ops.sample_filtered(logits.to(DEV), torch.arange(rows, dtype=torch.int32, device=DEV), rows, dparams,
                        torch.tensor([p.top_k for p in params], dtype=torch.int32, device=DEV), out)
    got = out.cpu().tolist()
    refs = [samplers[r].sample_host(logits[r].numpy().copy(), [], u=float(u[r])) for r in range(rows)]
    assert ops.SAMPLE_FILTERED_HOST not in got
    assert sum(a == b for a, b in zip(got, refs)) >= rows - 1, (got, refs)
    on_plateau = [r for r in range(rows) if float(logits[r, refs[r]]) == 1.5]
    assert len(on_plateau) >= 3                      # the case is met: draws that end among the equal logits
    for r in range(rows):
        assert got[r] == refs[r] or (float(logits[r, got[r]]) == float(logits[r, refs[r]]) and abs(got[r] - refs[r]) <= 1), (r, got[r], refs[r])


def test_sample_temperature_with_min_p(ops):
    """min-p in the walk down the ids: against the host's pipeline with the same uniform numbers."""
    from dynalm_b200.sampling import SamplingParams
    from dynalm_b200.sampling.sampler import Sampler
    g = torch.Generator(device="cpu").manual_seed(21)
    vocab, rows = 20011, 24
    logits = _peaked_logits(rows, vocab, g, 1.0)
    u = torch.rand(rows, generator=g, dtype=torch.float64)
    params = [SamplingParams(temperature=0.9, min_p=(0.0 if r % 3 == 0 else 0.02 * r)) for r in range(rows)]
    samplers = [Sampler(p) for p in params]
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.sample_temperature(logits.to(DEV), torch.full((rows,), 0.9, device=DEV), u.to(DEV), out,
                           cut_offset=torch.tensor([s.cut_offset for s in samplers], dtype=torch.float64, device=DEV))
    got = out.cpu().tolist()
    same = 0
    for r in range(rows):
        ref = samplers[r].sample_host(logits[r].numpy().copy(), [], u=float(u[r]))
        same += got[r] == ref
        if params[r].min_p > 0:
            cut = float(logits[r].max()) + samplers[r].cut_offset
            assert float(logits[r, got[r]]) >= cut
    assert same >= rows - 1


@pytest.mark.parametrize("dtype", DTYPES + ["tensor_cores"])
@pytest.mark.parametrize("heads,kvh,hd,page,window,splits", [(4, 2, 16, 16, 0, 1), (6, 2, 32, 16, 0, 3), (5, 1, 48, 16, 0, 4),
                                                               (3, 3, 80, 32, 0, 2), (8, 2, 128, 16, 40, 2),
                                                               (16, 2, 64, 16, 0, 5), (32, 8, 64, 16, 0, 8),
                                                               (4, 4, 256, 16, 0, 2), (4, 4, 64, 16, 7, 1),
                                                               (40, 2, 64, 16, 0, 3), (2, 1, 112, 64, 300, 6), (4, 2, 64, 16, 0, 12)])
def test_paged_attention_decode(ops, dtype, heads, kvh, hd, page, window, splits):
    """The split-KV kernel against the same reference as the plain kernel: requests of 1, 60, 700 and
    130 tokens in scattered pages, one row each at its last position, a far key that stands out,
    any number of splits (more splits than the short requests have keys)."""
    tc = dtype == "tensor_cores"
    if tc:
        dtype = torch.bfloat16
        if hd > 128:
            pytest.skip("the tensor-core variant holds head sizes up to 128")
    if dtype == torch.float32 and hd > 128:
        pytest.skip("the float32 instantiation holds head sizes up to 128")
    g = torch.Generator(device="cpu").manual_seed(10)
    lens = [1, 60, 700, 130]
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 5
    perm = torch.randperm(pages, generator=g)
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(pages, page, kvh, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    keys, vals = [], []
    nxt = 0
    for r, l in enumerate(lens):
        k = torch.randn(l, kvh, hd, generator=g).to(dtype)
        v = torch.randn(l, kvh, hd, generator=g).to(dtype)
        k[min(3, l - 1)] *= 4.0
        keys.append(k)
        vals.append(v)
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            nxt += 1
            n = min(page, l - b * page)
            kc[table[r, b], :n] = k[b * page:b * page + n]
            vc[table[r, b], :n] = v[b * page:b * page + n]
    order = [2, 0, 3, 1]
    req = torch.tensor(order, dtype=torch.int32)
    pos = torch.tensor([lens[r] - 1 for r in order], dtype=torch.int32)
    n = len(order)
    q = torch.randn(n, heads, hd, generator=g).to(dtype)
    q[0] = (keys[2][3, 0].float() * 0.5).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(n, heads * hd, dtype=dtype, device=DEV)
    scratch = torch.zeros(max(1, ops.decode_scratch_floats(n, heads, hd, splits)), dtype=torch.float32, device=DEV)
    ops.paged_attention_decode(q.reshape(n, heads * hd).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), pos.to(DEV),
                               req.to(DEV), out, scratch, heads, kvh, hd, page, scale, window, splits, tensor_cores=tc)
    got = out.double().cpu().reshape(n, heads, hd)
    for i, r in enumerate(order):
        ref = _attention_ref(q[i].double(), keys[r].double(), vals[r].double(), scale, window)
        err = (got[i] - ref).abs().max().item()
        assert err <= tol(dtype, 2), f"row {i} (request {r}): {err}"


@pytest.mark.parametrize("heads,kvh,hd,splits", [(32, 8, 64, 2), (32, 8, 64, 4), (8, 2, 128, 2), (12, 4, 64, 8), (6, 2, 32, 4), (3, 1, 128, 8), (8, 2, 128, 4)])
def test_paged_attention_decode_many_rows_in_clusters(ops, heads, kvh, hd, splits):
    """2, 4 and 8 key splits of a row are one thread-block cluster that merges in its first block's shared memory, at
    any number of rows: 30 rows over requests of 1 to 2,048 keys (many more clusters than SMs hold at once for the
    widest shape), the scratch left untouched; against float64."""
    page = 16
    g = torch.Generator(device="cpu").manual_seed(77 + hd + splits)
    lens = [700, 1, 130, 60, 333, 2048, 17, 129]
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 5
    perm = torch.randperm(pages, generator=g)
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(pages, page, kvh, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    keys, vals, nxt = [], [], 0
    for r, l in enumerate(lens):
        k = torch.randn(l, kvh, hd, generator=g).to(torch.bfloat16)
        v = torch.randn(l, kvh, hd, generator=g).to(torch.bfloat16)
        k[min(3, l - 1)] *= 4.0
        keys.append(k)
        vals.append(v)
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            nxt += 1
            n = min(page, l - b * page)
            kc[table[r, b], :n] = k[b * page:b * page + n]
            vc[table[r, b], :n] = v[b * page:b * page + n]
    order = [(5 * i) % len(lens) for i in range(30)]
    req = torch.tensor(order, dtype=torch.int32)
    pos = torch.tensor([lens[r] - 1 for r in order], dtype=torch.int32)
    q = torch.randn(len(order), heads, hd, generator=g).to(torch.bfloat16)
    q[0] = (keys[order[0]][3, 0].float() * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(len(order), heads * hd, dtype=torch.bfloat16, device=DEV)
    scratch = torch.full((ops.decode_scratch_floats(len(order), heads, hd, splits),), float("nan"), dtype=torch.float32, device=DEV)
    ops.paged_attention_decode(q.reshape(len(order), heads * hd).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV), pos.to(DEV),
                               req.to(DEV), out, scratch, heads, kvh, hd, page, scale, 0, splits, tensor_cores=True)
    assert bool(torch.isnan(scratch).all()), "the splits were expected to merge inside their cluster"
    got = out.double().cpu().reshape(len(order), heads, hd)
    for i, r in enumerate(order):
        ref = _attention_ref(q[i].double(), keys[r].double(), vals[r].double(), scale, 0)
        err = (got[i] - ref).abs().max().item()
        assert err <= tol(torch.bfloat16, 2), f"row {i} (request {r}): {err}"


@pytest.mark.parametrize("heads,kvh,hd,page,window", [(4, 2, 16, 16, 0), (6, 2, 32, 16, 0), (5, 1, 48, 16, 0),
                                                        (3, 3, 80, 32, 0), (8, 2, 128, 16, 40), (32, 8, 64, 16, 0),
                                                        (4, 4, 64, 16, 7), (2, 1, 112, 16, 100), (4, 2, 96, 64, 0)])
def test_paged_attention_prefill(ops, heads, kvh, hd, page, window):
    """The mma.sync flash kernel; see _check_prefill_kernel."""
    _check_prefill_kernel(ops.paged_attention_prefill, heads, kvh, hd, page, window)


@pytest.mark.parametrize("heads,kvh,hd,page,window", [(32, 8, 64, 16, 0), (4, 4, 64, 16, 7), (8, 2, 128, 16, 40),
                                                        (6, 2, 128, 32, 0), (3, 1, 64, 64, 300), (2, 2, 128, 16, 129)])
def test_paged_attention_prefill_tcgen05(ops, heads, kvh, hd, page, window):
    """The tcgen05 flash kernel (head sizes 64 and 128) on the same mixed batch, twice in a row (tensor memory
    is freed and taken again), with no timeout recorded."""
    for _ in range(2):
        _check_prefill_kernel(ops.paged_attention_prefill_tcgen05, heads, kvh, hd, page, window)
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("heads,kvh,hd,page,window", [(4, 2, 64, 16, 0), (2, 1, 128, 64, 0), (2, 2, 64, 32, 1000)])
def test_paged_attention_prefill_tcgen05_long_context(ops, heads, kvh, hd, page, window):
    """A request of 3,000 keys (47 tiles of 64: many rounds of the kernel's two S buffers and of its K/V stages): a
    full 128-row tile at its end and a 70-row one in the middle, with a key far above the running maximum late in the
    context (rows that see it rescale their sums after dozens of tiles) and one early; against float64."""
    g = torch.Generator(device="cpu").manual_seed(hd + page)
    L = 3000
    k = torch.randn(L, kvh, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(L, kvh, hd, generator=g).to(torch.bfloat16)
    k[5] *= 4.0
    k[2700] *= 6.0
    n_pages = -(-L // page)
    perm = torch.randperm(n_pages + 3, generator=g)
    table = perm[:n_pages].to(torch.int32).view(1, n_pages).contiguous()
    kc = torch.zeros(n_pages + 3, page, kvh, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for b in range(n_pages):
        n = min(page, L - b * page)
        kc[table[0, b], :n] = k[b * page:b * page + n]
        vc[table[0, b], :n] = v[b * page:b * page + n]
    runs = [(L - 128, 128), (1500, 70)]                       # (first position, rows)
    rows = [p0 + i for p0, n in runs for i in range(n)]
    tiles, row0 = [], 0
    for p0, n in runs:
        tiles.append((0, row0, n, p0))
        row0 += n
    q = torch.randn(len(rows), heads, hd, generator=g).to(torch.bfloat16)
    for i, p in enumerate(rows):
        if i % 3 == 0:
            q[i] = (k[2700, 0].float() * 0.2).to(torch.bfloat16)       # sees the late key (if its position is past it)
        if i % 3 == 1:
            q[i] = (k[5, 0].float() * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(len(rows), heads * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill_tcgen05(q.reshape(len(rows), heads * hd).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV),
                                        torch.tensor(tiles, dtype=torch.int32).to(DEV), len(tiles), out, heads, kvh, hd, page,
                                        scale, window)
    assert ops.gemm_tcgen05_status() == 0, "a wait inside the kernel timed out"
    got = out.double().cpu().reshape(len(rows), heads, hd)
    for i, p in enumerate(rows):
        ref = _attention_ref(q[i].double(), k[:p + 1].double(), v[:p + 1].double(), scale, window)
        err = (got[i] - ref).abs().max().item()
        assert err <= 2.5e-2, f"row {i} (position {p}): {err}"


@pytest.mark.parametrize("heads,kvh,hd,page,window", [(4, 2, 64, 16, 0), (3, 1, 128, 32, 0), (2, 2, 64, 16, 900)])
def test_paged_attention_prefill_tcgen05_keys_dealt_over_blocks(ops, heads, kvh, hd, page, window):
    """The keys of a query tile dealt over several blocks that leave their parts in scratch, the last one adding them
    up: a 128-row tile at the end of 3,000 keys in 3 parts, a 70-row tile in the middle in 2, a short tile whole;
    twice over the same counters; against float64 and against the same tiles whole."""
    g = torch.Generator(device="cpu").manual_seed(3 * hd + page)
    L = 3000
    k = torch.randn(L, kvh, hd, generator=g).to(torch.bfloat16)
    v = torch.randn(L, kvh, hd, generator=g).to(torch.bfloat16)
    k[5] *= 4.0
    k[2700] *= 6.0
    n_pages = -(-L // page)
    perm = torch.randperm(n_pages + 3, generator=g)
    table = perm[:n_pages].to(torch.int32).view(1, n_pages).contiguous()
    kc = torch.zeros(n_pages + 3, page, kvh, hd, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    for b in range(n_pages):
        n = min(page, L - b * page)
        kc[table[0, b], :n] = k[b * page:b * page + n]
        vc[table[0, b], :n] = v[b * page:b * page + n]
    runs = [(L - 128, 128, 3), (1500, 70, 2), (40, 9, 1)]                 # (first position, rows, parts)
    rows = [p0 + i for p0, n, _ in runs for i in range(n)]
    whole, dealt, words, row0, record = [], [], [], 0, 0
    for p0, n, parts in runs:
        whole.append((0, row0, n, p0))
        for p in range(parts):
            dealt.append((0, row0, n, p0))
            words.append(0 if parts == 1 else (p | parts << 8 | record << 16))
        record += parts if parts > 1 else 0
        row0 += n
    q = torch.randn(len(rows), heads, hd, generator=g).to(torch.bfloat16)
    for i, p in enumerate(rows):
        if i % 3 == 0:
            q[i] = (k[2700, 0].float() * 0.2).to(torch.bfloat16)
        if i % 3 == 1:
            q[i] = (k[5, 0].float() * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(hd)
    dev = [t.to(DEV) for t in (q.reshape(len(rows), heads * hd), kc, vc, table)]
    ref_out = torch.zeros(len(rows), heads * hd, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention_prefill_tcgen05(*dev, torch.tensor(whole, dtype=torch.int32).to(DEV), len(whole), ref_out, heads, kvh, hd,
                                        page, scale, window)
    partial = torch.full((record * heads * (hd + 2) * 128,), float("nan"), dtype=torch.float32, device=DEV)
    counters = torch.zeros(record * heads, dtype=torch.int32, device=DEV)
    for again in range(2):
        out = torch.zeros_like(ref_out)
        ops.paged_attention_prefill_tcgen05(*dev, torch.tensor(dealt, dtype=torch.int32).to(DEV), len(dealt), out, heads, kvh, hd,
                                            page, scale, window, unit_parts=torch.tensor(words, dtype=torch.int32).to(DEV),
                                            partial=partial, counters=counters)
        assert ops.gemm_tcgen05_status() == 0, "a wait inside the kernel timed out"
        assert int(counters.abs().sum()) == 0, "the counters are left at zero"
        got = out.double().cpu().reshape(len(rows), heads, hd)
        for i, p in enumerate(rows):
            ref = _attention_ref(q[i].double(), k[:p + 1].double(), v[:p + 1].double(), scale, window)
            err = (got[i] - ref).abs().max().item()
            assert err <= 2.5e-2, f"pass {again} row {i} (position {p}): {err}"
        assert (out.float() - ref_out.float()).abs().max().item() <= 2e-2       # the same tiles whole: bf16 rounding apart
        assert torch.equal(out[128 + 70:], ref_out[128 + 70:])                   # the whole tile among them: the same bits


def test_paged_attention_prefill_tcgen05_refuses_other_shapes(ops):
    q = torch.zeros(4, 2 * 48, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(3, 16, 1, 48, dtype=torch.bfloat16, device=DEV)
    tiles = torch.tensor([[0, 0, 4, 0]], dtype=torch.int32, device=DEV)
    table = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(Exception, match="head_dim 48"):
        ops.paged_attention_prefill_tcgen05(q, kc, kc.clone(), table, tiles, 1, torch.zeros_like(q), 2, 1, 48, 16, 0.1, 0)
    q = torch.zeros(4, 2 * 64, dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros(6, 8, 1, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="page size 8"):
        ops.paged_attention_prefill_tcgen05(q, kc, kc.clone(), table, tiles, 1, torch.zeros_like(q), 2, 1, 64, 8, 0.1, 0)


def _check_prefill_kernel(run, heads, kvh, hd, page, window):
    """A flash kernel on a mixed batch: a decode row, a 210-row portion that starts in the middle of a
    page and of a key tile, a 5-row run, another decode row and a 64-row portion from position 0; an
    early key stands out for some rows and a late one (far above the running maximum) for others;
    queries padded inside a wider row (as q inside qkv)."""
    dtype = torch.bfloat16
    g = torch.Generator(device="cpu").manual_seed(12)
    lens = [60, 700, 130, 64]
    max_blocks = -(-max(lens) // page)
    pages = sum(-(-l // page) for l in lens) + 5
    perm = torch.randperm(pages, generator=g)
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(pages, page, kvh, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    keys, vals = [], []
    nxt = 0
    for r, l in enumerate(lens):
        k = torch.randn(l, kvh, hd, generator=g).to(dtype)
        v = torch.randn(l, kvh, hd, generator=g).to(dtype)
        k[3] *= 4.0
        k[l - 12] *= 5.0
        keys.append(k)
        vals.append(v)
        for b in range(-(-l // page)):
            table[r, b] = perm[nxt]
            nxt += 1
            n = min(page, l - b * page)
            kc[table[r, b], :n] = k[b * page:b * page + n]
            vc[table[r, b], :n] = v[b * page:b * page + n]
    if window > 0:
        # pages wholly behind the window of the first row of each run are not there any more
        pass
    runs = [(0, 59, 1), (1, 700 - 210, 210), (2, 100, 5), (2, 129, 1), (3, 0, 64)]      # (request, first position, rows)
    rows = [(r, p0 + i) for r, p0, n in runs for i in range(n)]
    tiles = []
    row0 = 0
    for r, p0, n in runs:
        for t0 in range(0, n, 128):
            tiles.append((r, row0 + t0, min(128, n - t0), p0 + t0))
        row0 += n
    n = len(rows)
    q = torch.randn(n, heads, hd, generator=g).to(dtype)
    for i, (r, p) in enumerate(rows):
        if i % 3 == 0:
            q[i, :, :] = (keys[r][3, 0].float() * 0.5).to(dtype)
        if i % 3 == 1:
            q[i, :, :] = (keys[r][lens[r] - 12, 0].float() * 0.2).to(dtype)
    wide = torch.zeros(n, heads * hd + 2 * kvh * hd, dtype=dtype)
    wide[:, :heads * hd] = q.reshape(n, heads * hd)
    wide = wide.to(DEV)
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(n, heads * hd, dtype=dtype, device=DEV)
    run(wide[:, :heads * hd], kc.to(DEV), vc.to(DEV), table.to(DEV),
        torch.tensor(tiles, dtype=torch.int32).to(DEV), len(tiles), out, heads, kvh, hd, page, scale, window)
    got = out.double().cpu().reshape(n, heads, hd)
    for i, (r, p) in enumerate(rows):
        ref = _attention_ref(q[i].double(), keys[r][:p + 1].double(), vals[r][:p + 1].double(), scale, window)
        err = (got[i] - ref).abs().max().item()
        assert err <= 2.5e-2, f"row {i} (request {r}, position {p}): {err}"
    # a row's result does not depend on where its portion was cut: the 210-row run again as 7 + 203 rows
    runs2 = [(1, 700 - 210, 7), (1, 700 - 203, 203)]
    tiles2, row0 = [], 1
    for r, p0, m in runs2:
        for t0 in range(0, m, 64):
            tiles2.append((r, row0 + t0, min(64, m - t0), p0 + t0))
        row0 += m
    out2 = torch.zeros_like(out)
    run(wide[:, :heads * hd], kc.to(DEV), vc.to(DEV), table.to(DEV),
        torch.tensor(tiles2, dtype=torch.int32).to(DEV), len(tiles2), out2, heads, kvh, hd, page, scale, window)
    assert torch.equal(out2[1:211], out[1:211])


@pytest.mark.parametrize("M,N,K", [(1, 3072, 2048), (8, 499, 80), (7, 130, 200), (16, 96, 1000), (9, 48, 64), (33, 250, 264),
                                   (64, 160, 96), (3, 17, 8)])
def test_gemm_skinny(ops, M, N, K):
    g = torch.Generator(device="cpu").manual_seed(13)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(DEV, torch.bfloat16)
    ref = x.double() @ w.double().T
    scale = ref.abs().max().item()
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(x, w, out32, "store", 0.5)
    assert (out32.double() - 0.5 * ref).abs().max() <= 1e-5 * scale
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(x, w, out16)
    assert (out16.double() - ref).abs().max() <= 1e-2 * scale
    # x as a view with a wider row (q inside qkv), K split over 3 blocks, parts added by the consumer
    wide = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    parts = torch.empty(3, M, N, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(wide[:, :K], w, parts)
    assert (parts.sum(0).double() - ref).abs().max() <= 1e-5 * scale
    # fused SwiGLU: w = [gate; up]
    if N % 2 == 0:
        act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        ops.gemm_skinny(x, w, act, "swiglu")
        gate, up = ref[:, :N // 2], ref[:, N // 2:]
        want = gate * torch.sigmoid(gate) * up
        assert (act.double() - want).abs().max() <= 1e-2 * max(1.0, want.abs().max().item())
    # the consumer adds the parts in order
    resid = torch.randn(M, N, generator=g).to(DEV)
    wn = torch.ones(N, device=DEV)
    normed = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    r2 = resid.clone()
    ops.rmsnorm(r2, wn, 1e-5, normed, delta=parts, delta_scale=1.0)
    assert (r2.double() - (resid.double() + ref)).abs().max() <= 2e-5 * max(1.0, scale)


@pytest.fixture(params=["alone", "pairs"])
def tile_sharing(request, ops, monkeypatch):
    """Runs a test with the tcgen05 product in which every block loads its own operands, and with the one in which
    two blocks share each tile of W (forced for every size, also those for which the dispatcher would not use it)."""
    monkeypatch.setattr(ops, "PAIRS_MIN_WAVES", 0 if request.param == "pairs" else 1 << 30)
    return request.param


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (100, 264, 200), (300, 1000, 136), (17, 48, 8),
                                   (2048, 3072, 2048), (513, 4096, 1024)])
def test_gemm_tcgen05(ops, tile_sharing, M, N, K):
    """The tcgen05 / TMEM / TMA matrix product against an fp64 reference: tiles that end inside M, N
    and K (an odd number of row blocks leaves a pair's second block without rows), all three epilogues, and an
    operand that is a view with a wider row."""
    g = torch.Generator(device="cpu").manual_seed(14)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(DEV, torch.bfloat16)
    ref = x.double() @ w.double().T
    scale = ref.abs().max().item()
    out16 = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(x, w, out16)
    assert ops.gemm_tcgen05_status() == 0, "a wait inside the kernel timed out"
    assert (out16.double() - ref).abs().max() <= 1e-2 * scale
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(x, w, out32, "store", 0.5)
    assert (out32.double() - 0.5 * ref).abs().max() <= 2e-5 * scale
    wide = torch.zeros(M, K + 40, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    out32b = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(wide[:, :K], w, out32b)
    assert (out32b.double() - ref).abs().max() <= 2e-5 * scale
    if N % 16 == 0:
        act = torch.empty(M, N // 2, dtype=torch.bfloat16, device=DEV)
        ops.gemm_tcgen05(x, w, act, "swiglu")
        gate, up = ref[:, :N // 2], ref[:, N // 2:]
        want = gate * torch.sigmoid(gate) * up
        assert (act.double() - want).abs().max() <= 1e-2 * max(1.0, want.abs().max().item())
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("rows,heads,kvh,hd,K,page", [(8, 32, 8, 64, 2048, 16), (1, 4, 4, 16, 80, 16), (13, 6, 2, 128, 264, 32),
                                                      (16, 5, 1, 48, 1000, 16), (300, 32, 8, 64, 512, 16),
                                                      (133, 5, 1, 128, 200, 32), (1000, 6, 3, 64, 72, 16)])
def test_gemm_qkv_rope_matches_the_separate_kernels(ops, tile_sharing, rows, heads, kvh, hd, K, page):
    """Projection + rotation + cache write in one kernel (weight-streaming up to 16 rows, tcgen05 beyond) against
    the plain product followed by rope_cache_write:
    the same q and the same cache pages (positions in the middle of pages, requests in shuffled rows)."""
    g = torch.Generator(device="cpu").manual_seed(5)
    width = (heads + 2 * kvh) * hd
    x = (torch.randn(rows, K, generator=g) * 0.5).bfloat16().to(DEV)
    w = (torch.randn(width, K, generator=g) / math.sqrt(K)).bfloat16().to(DEV)
    inv_freq = (10000.0 ** (-torch.arange(0, hd, 2, dtype=torch.float32) / hd)).to(DEV)
    n_req = min(rows, 16)                      # row r belongs to request r % n_req, at a position of its own
    span = 90 * -(-rows // n_req)
    positions = torch.tensor([(37 * (r % n_req) + 5) % 90 + 90 * (r // n_req) for r in range(rows)], dtype=torch.int32,
                             device=DEV)
    row_request = torch.tensor([(r * 7) % n_req if rows <= 16 else r % n_req for r in range(rows)], dtype=torch.int32,
                               device=DEV)
    if rows <= 16:
        positions = torch.tensor([(37 * r + 5) % 90 for r in range(rows)], dtype=torch.int32, device=DEV)
    max_blocks = -(-span // page)
    table = torch.randperm(n_req * max_blocks, generator=g).to(torch.int32).view(n_req, max_blocks).to(DEV)
    pages = n_req * max_blocks

    def caches():
        return (torch.zeros(pages, page, kvh, hd, dtype=torch.bfloat16, device=DEV),
                torch.zeros(pages, page, kvh, hd, dtype=torch.bfloat16, device=DEV))
    k_ref, v_ref = caches()
    qkv_ref = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    if rows <= 16:
        ops.gemm_skinny(x, w, qkv_ref)
    else:
        ops.gemm_tcgen05(x, w, qkv_ref)
    ops.rope_cache_write(qkv_ref, positions, row_request, table, k_ref, v_ref, inv_freq, hd, 0.5, heads, kvh, hd, page)
    k_got, v_got = caches()
    qkv_got = torch.zeros(rows, width, dtype=torch.bfloat16, device=DEV)
    ops.gemm_qkv_rope(x, w, qkv_got, positions, row_request, table, k_got, v_got, inv_freq, 0.5, heads, kvh, hd, page)
    q_ref, q_got = qkv_ref[:, :heads * hd].float(), qkv_got[:, :heads * hd].float()
    assert (q_ref - q_got).abs().max().item() <= 1e-2 * q_ref.abs().max().item()
    assert (k_ref.float() - k_got.float()).abs().max().item() <= 1e-2 * k_ref.float().abs().max().item()
    assert torch.equal(v_ref, v_got)
    assert k_got.abs().sum().item() > 0 and (k_got != 0).sum().item() == rows * kvh * hd
    if rows > 16:
        # the same with the step's (cos, sin) pairs computed once beforehand: the same bits
        angles = torch.zeros(rows, hd // 2, 2, dtype=torch.float32, device=DEV)
        ops.rope_angles(positions, inv_freq, 0.5, rows, angles)
        k2, v2 = caches()
        qkv2 = torch.zeros_like(qkv_got)
        ops.gemm_qkv_rope(x, w, qkv2, positions, row_request, table, k2, v2, inv_freq, 0.5, heads, kvh, hd, page, angles)
        assert torch.equal(qkv2[:, :heads * hd], qkv_got[:, :heads * hd]) and torch.equal(k2, k_got) and torch.equal(v2, v_got)
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("M,N,K", [(8, 3072, 2048), (1, 499 * 2, 80), (16, 256, 64), (17, 130, 200), (33, 1000, 264),
                                   (64, 2048, 1024), (40, 96, 8), (64, 640, 4096)])
def test_gemm_stream(ops, M, N, K):
    """The tcgen05 weight-streaming product (up to 64 rows, computed transposed) against an fp64 reference: tiles that
    end inside N and K, every row count class, bf16 / fp32 / scaled output, K splits with an empty split, SwiGLU."""
    g = torch.Generator(device="cpu").manual_seed(15)
    x = torch.randn(M, K, generator=g).to(DEV, torch.bfloat16)
    w = torch.randn(N, K, generator=g).to(DEV, torch.bfloat16)
    ref = x.double() @ w.double().T
    scale = ref.abs().max().item()
    out16 = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_stream(x, w, out16)
    assert ops.gemm_tcgen05_status() == 0, "a wait inside the kernel timed out"
    assert (out16.double() - ref).abs().max() <= 1e-2 * scale
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_stream(x, w, out32, "store", 0.5)
    assert (out32.double() - 0.5 * ref).abs().max() <= 2e-5 * scale
    for parts in (2, 5, 7):
        part = torch.full((parts, M, N), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_stream(x, w, part)
        assert (part.double().sum(0) - ref).abs().max() <= 2e-5 * scale, parts
    wide = torch.zeros(M, K + 24, dtype=torch.bfloat16, device=DEV)
    wide[:, :K] = x
    out32b = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_stream(wide[:, :K], w, out32b)
    assert (out32b.double() - ref).abs().max() <= 2e-5 * scale
    act = torch.full((M, N // 2), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.gemm_stream(x, w, act, "swiglu")
    gate, up = ref[:, :N // 2], ref[:, N // 2:]
    want = gate * torch.sigmoid(gate) * up
    assert (act.double() - want).abs().max() <= 1e-2 * max(1.0, want.abs().max().item())
    assert ops.gemm_tcgen05_status() == 0


@pytest.mark.parametrize("rows,N,K", [(1, 499, 64), (5, 128256, 256), (8, 4099, 2048), (8, 16, 8)])
def test_gemm_argmax_matches_argmax_of_the_product(ops, rows, N, K):
    """The product whose epilogue keeps only the place of each row's largest output gives what argmax gives on the
    logits the same kernel writes (the sums are the same, so the choice is exact), ties going to the lowest index."""
    g = torch.Generator(device="cpu").manual_seed(rows * 1000 + N)
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    if N > 40:
        w[37] = w[11]                      # two equal outputs in every row ...
        w[11] *= 0
        w[37] *= 0
        w[11, 0], w[37, 0] = 60.0, 60.0    # ... made the largest wherever x[r, 0] > 0
    w = w.to(DEV)
    logits = torch.empty(rows, N, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(x, w, logits, "store", 0.5)
    want = torch.empty(rows, dtype=torch.int32, device=DEV)
    ops.argmax(logits, want)
    got = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
    scratch = torch.empty(2 * rows * -(-N // 16), dtype=torch.float32, device=DEV)
    status = torch.full((1,), 7, dtype=torch.int32, device=DEV)
    ops.gemm_argmax(x, w, got, scratch, 0.5, status_to=status)
    assert got.cpu().tolist() == want.cpu().tolist()
    assert int(status.item()) == ops.gemm_tcgen05_status(DEV)
    assert 37 not in got.cpu().tolist()         # of the two equal outputs the lower index
    if N > 40 and K <= 256:
        assert any(float(x[r, 0]) > 0.5 and int(got[r]) == 11 for r in range(rows)) or not any(float(x[r, 0]) > 0.5 for r in range(rows))


def test_decode_tile_keys_agree_with_the_kernel(ops):
    """The plan counts a row's keys in the kernel's tiles: the table on the Python side is the kernel's."""
    import ctypes
    from dynalm_b200.kernels import lib
    f = lib.load("attention_decode").dl_paged_attention_decode_tile
    f.argtypes, f.restype = [ctypes.c_int], ctypes.c_int
    for hd in range(16, 129, 16):
        assert ops.decode_tile_keys(hd) == f(hd), hd



@pytest.mark.parametrize("heads,kvh,hd,window", [(8, 2, 64, 0), (6, 2, 32, 0), (3, 1, 128, 0), (32, 8, 64, 0), (4, 4, 80, 37)])
def test_planned_decode_attention(ops, heads, kvh, hd, window, monkeypatch):
    """The decode kernel with the keys dealt into units by the host, on requests of very different lengths (one long,
    some of a few keys, one of a single key), twice in a row over the same counters and scratch: against float64."""
    from dynalm_b200.engine.step import StepShape
    from dynalm_b200.kernels import attention as fast
    from dynalm_b200.kernels.attention import PART_CAP, DecodeUnits
    monkeypatch.setattr(fast, "PLANNED_MIN_ROWS", 1)        # (the engine plans from a dozen rows on; the kernel takes any)
    page = 16
    g = torch.Generator(device="cpu").manual_seed(heads * 100 + hd)
    chunks = kvh * -(-(heads // kvh) // 16)
    plan = DecodeUnits(chunks, ops.decode_tile_keys(hd), window)
    for lens in ([3000, 1, 77, 640, 33, 129, 2048, 15], [500, 4100]):
        rows = len(lens)
        max_blocks = -(-max(lens) // page)
        pages = sum(-(-l // page) for l in lens) + 3
        perm = torch.randperm(pages, generator=g)
        table = torch.full((rows, max_blocks), -1, dtype=torch.int32)
        kc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
        vc = torch.randn(pages, page, kvh, hd, generator=g).to(torch.bfloat16)
        keys, vals, nxt = [], [], 0
        for r, l in enumerate(lens):
            mine = [int(p) for p in perm[nxt:nxt + -(-l // page)]]
            nxt += len(mine)
            table[r, :len(mine)] = torch.tensor(mine, dtype=torch.int32)
            keys.append(kc[mine].reshape(-1, kvh, hd)[:l])
            vals.append(vc[mine].reshape(-1, kvh, hd)[:l])
        q = torch.randn(rows, heads * hd, generator=g).to(torch.bfloat16)
        q[0, :hd] *= 4          # one far key of the long request stands out: a unit that is skipped shows
        pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
        req = torch.arange(rows, dtype=torch.int32)
        host = np.zeros(plan.ints(0, rows), dtype=np.int32)
        units, n_rows = plan.fill(host, StepShape([1] * rows, list(range(rows)), [l - 1 for l in lens], list(range(rows)), rows))
        assert n_rows == rows and units <= plan.unit_cap(rows)
        d = [t.to(DEV) for t in (q, kc, vc, table, pos, req)]
        out = torch.zeros(rows, heads * hd, dtype=torch.bfloat16, device=DEV)
        scratch = torch.full((rows * heads * PART_CAP * (hd + 2),), float("nan"), device=DEV)
        counters = torch.zeros(rows * chunks, dtype=torch.int32, device=DEV)
        plan_dev = torch.from_numpy(host).to(DEV)
        scale = hd ** -0.5
        for again in range(2):
            out.zero_()
            ops.paged_attention_decode_planned(d[0], d[1], d[2], d[3], d[4], d[5], out, scratch, counters, plan_dev,
                                               plan.unit_cap(rows), PART_CAP, heads, kvh, hd, page, scale, window)
            got = out.float().cpu().view(rows, heads, hd)
            assert int(counters.abs().sum()) == 0
            for i in range(rows):
                ref = _attention_ref(q[i].view(heads, hd).double(), keys[i].double(), vals[i].double(), scale, window)
                err = (got[i] - ref).abs().max().item()
                assert err <= 2.5e-2, f"lens {lens} row {i} pass {again}: {err}"
