"""The Llama 3.2 1B and 3B layer sizes (2 of their layers, the full vocabulary, tied embeddings, llama3 RoPE scaling;
head size 64 in groups of four, head size 128 in groups of three) with random weights, against the plain implementation: whole prompts, portions, and mixed steps of up to four
live requests in a pool so small that pages are used again. At these sizes the bfloat16 engine runs what the tiny
configurations cannot reach: the tcgen05 products (also the one in which two blocks share tiles of W, from 1,184
rows), the tcgen05 prompt attention over many query tiles (in the 3,500-token prompt brought in portions of 512 also
with the keys of a query tile dealt over several blocks), and the library product for the row counts in between.

32-bit: logits within 1e-4 of each row's largest logit. bfloat16: what the reference asks of its own GPU path
against 32-bit, a mean KL divergence of at most 0.0025 and the same most likely token in at least 99 rows of 100
(dynalm/benchmarks/bench_gpu_accuracy.cpp:91-92), here against the plain implementation on the same bfloat16
weights."""

import json
import os

import numpy as np
import pytest
import torch

from plain_llama import PlainLlama
from replay_util import Plan, compare, kl_and_top1, plan_mixed, random_requests, run_plan_in_process

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
CFG_3B = dict(CFG, hidden_size=3072, num_attention_heads=24, head_dim=128)
SHAPES = {"1B": CFG, "3B": CFG_3B}
LENGTHS = [300, 170, 230, 129, 90, 200]
LONG = 1300
LONG_WANT = list(range(LONG - 6, LONG))
# A prompt long enough for the keys of its last query tiles to be dealt over several blocks (from 48 key tiles of
# 64), brought in portions of 512; wanted: rows of the first portion with dealt keys and of the last.
FAR = 3500
FAR_PORTION = 512
FAR_WANT = [3071, 3072, 3199, 3327, 3328] + list(range(FAR - 4, FAR))


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request):
    return request.param


@pytest.fixture(scope="module")
def folder(tmp_path_factory, shape):
    from dynalm_b200.registry import find_architecture
    from dynalm_b200.weights import random_tensors, write_safetensors
    CFG = SHAPES[shape]
    d = str(tmp_path_factory.mktemp(f"shape_{shape}"))
    arch = find_architecture(CFG)
    t = random_tensors(arch.plan(arch.read_config(CFG)), 0, torch.bfloat16)
    # random N(0, 0.02) weights give nearly flat logits; a wider embedding makes the distribution peaked
    # enough for the most likely token and the KL divergence to mean something
    t["model.embed_tokens.weight"] = (t["model.embed_tokens.weight"].float() * 8).to(torch.bfloat16)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(CFG, f)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    return d


def _plans():
    reqs = random_requests(CFG["vocab_size"], LENGTHS, seed=3)
    long = random_requests(CFG["vocab_size"], [LONG], seed=4)["r0"]
    reqs["long"] = long
    whole = Plan()
    whole.add([("long", long, 0, LONG_WANT)], end=["long"])
    cut = Plan()
    pos = 0
    for n in (700, 513, 2, 85):
        cut.add([("long", long[pos:pos + n], pos, [w - pos for w in LONG_WANT if pos <= w < pos + n])],
                end=["long"] if pos + n == LONG else [])
        pos += n
    short = {r: t for r, t in reqs.items() if r != "long"}
    mixed = plan_mixed(short, seed=8, max_live=4, decode_tail=6, sizes=(2, 33, 130, 64, 257))
    far = random_requests(CFG["vocab_size"], [FAR], seed=5)["r0"]
    reqs["far"] = far
    portions = Plan()
    for pos in range(0, FAR, FAR_PORTION):
        n = min(FAR_PORTION, FAR - pos)
        portions.add([("far", far[pos:pos + n], pos, [w - pos for w in FAR_WANT if pos <= w < pos + n])],
                     end=["far"] if pos + n == FAR else [])
    return reqs, {"whole": whole, "cut": cut, "mixed": mixed, "portions": portions}


@pytest.fixture(scope="module")
def plain(folder):
    """request -> {position: plain logits row}, for the positions that some plan wants."""
    reqs, plans = _plans()
    wanted = {r: set() for r in reqs}
    for plan in plans.values():
        for rows in plan.rows.values():
            for r, pos in rows:
                wanted[r].add(pos)
    model = PlainLlama(folder)
    out = {}
    for r, toks in reqs.items():
        places = sorted(wanted[r])
        got = model.logits(toks, rows=places).astype(np.float32)
        out[r] = {pos: got[i] for i, pos in enumerate(places)}
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layer_shapes_against_plain(dtype, shape, folder, plain):
    from dynalm_b200.engine import build
    from dynalm_b200.kernels import gemm
    _, plans = _plans()
    for what, plan in plans.items():
        need = plan.max_live_tokens(64)
        library_before = gemm.LIBRARY_CALLS
        built = build(folder, dtype=dtype, kv_tokens=need, max_batch_tokens=1408, max_requests=4,
                      context=4096 if what == "portions" else 2048)
        got = run_plan_in_process(built.step_fn, plan)
        assert built.cache.free_pages == built.cache.num_pages
        if what == "portions" and dtype == "bfloat16":
            dealt = [key for key in built.runtime._buffers if str(key[0]).startswith("attn_tile_parts_")]
            assert dealt, "no query tile had its keys dealt over several blocks"
        kl, top1 = kl_and_top1(plan, got, plain, near_tie=1e-4 if dtype == "float32" else 0.05)
        if dtype == "float32":
            worst = compare(plan, got, plain, 0.0, 1e-4, f"{shape}/{dtype}/{what}")
            assert kl <= 1e-9 and top1 == 1.0
        else:
            worst = compare(plan, got, plain, 0.0, 5e-2, f"{shape}/{dtype}/{what}")
            # (rows whose two largest plain logits lie within 0.05 of each other are not counted against it; of the
            # others a few in a thousand still change places under bfloat16 rounding at this logit scale)
            assert kl <= 0.0025 and top1 >= 0.99, f"{shape}/{dtype}/{what}: mean KL {kl:.3g}, top-1 agreement {top1:.4f}"
            if what == "mixed":
                assert gemm.LIBRARY_CALLS > library_before, "no product took the path of 17 to 127 rows"
        print(f"{shape} {dtype} {what}: steps {len(plan.steps)} pool {need} worst {worst:.3g} KL {kl:.3g} top-1 {top1:.4f}")
        del built
        torch.cuda.empty_cache()
