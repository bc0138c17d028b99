"""Random Llama configurations (head sizes in steps of 16, any heads and groups, widths and vocabularies that are no
power of two, every rope scaling, partial rotary widths, multipliers, pages of 16 to 64 tokens) replayed whole, in
portions and mixed, in 32-bit and in bfloat16, against the plain implementation: what the dispatchers choose for
a shape must never change a result beyond rounding."""

import tempfile

import numpy as np
import pytest
import torch

from plain_llama import PlainLlama
from replay_util import compare, plan_chunks, plan_mixed, plan_whole, random_requests, run_plan_in_process

pytestmark = pytest.mark.gpu

TOL = {"float32": (2e-5, 2e-5), "bfloat16": (2e-2, 4e-2)}


def random_config(rng) -> dict:
    kv_heads = int(rng.choice([1, 2, 3, 4]))
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
           "vocab_size": int(rng.choice([97, 256, 301, 512, 1000])),
           "hidden_size": int(rng.choice([40, 72, 100, 128, 136, 200, 264])),
           "intermediate_size": int(rng.choice([48, 100, 172, 256, 344])),
           "num_hidden_layers": int(rng.choice([1, 2, 3])),
           "num_attention_heads": kv_heads * int(rng.choice([1, 2, 3, 4, 5])), "num_key_value_heads": kv_heads,
           "head_dim": int(rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128])), "max_position_embeddings": 1024,
           "rms_norm_eps": float(rng.choice([1e-5, 1e-6, 3e-5])), "rope_theta": float(rng.choice([10000.0, 500000.0])),
           "tie_word_embeddings": bool(rng.rand() < 0.5)}
    r = rng.rand()
    if r < 0.3:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                               "original_max_position_embeddings": 64}
    elif r < 0.45:
        cfg["rope_scaling"] = {"type": "linear", "factor": 2.0}
    if rng.rand() < 0.25:
        cfg["partial_rotary_factor"] = 0.5
    if rng.rand() < 0.2:
        cfg.update({"embedding_multiplier": 2.0, "residual_multiplier": 0.7, "attention_multiplier": 0.15,
                    "logits_scaling": 3.0})
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_random_configuration(seed):
    from dynalm_b200.engine import build
    from dynalm_b200.weights import write_model_folder
    rng = np.random.RandomState(1000 + seed)
    cfg = random_config(rng)
    with tempfile.TemporaryDirectory() as folder:
        write_model_folder(folder, cfg, seed, torch.float32)
        model = PlainLlama(folder)
        lens = [int(x) for x in rng.randint(1, 400, size=rng.randint(3, 7))]
        reqs = random_requests(cfg["vocab_size"], lens, seed=seed)
        plain = {r: model.logits(t) for r, t in reqs.items()}
        for dtype in ("float32", "bfloat16"):
            plans = {"mixed": plan_mixed(reqs, seed=seed, max_live=int(rng.randint(1, 5)), decode_tail=int(rng.randint(1, 40)),
                                         sizes=(2, 3, 5, 7, 16, 24, 64, 130, 200)),
                     "chunks": plan_chunks(reqs, [17, 130, 2, 64, 300, 5]), "whole": plan_whole(reqs)}
            for what, plan in plans.items():
                need = plan.max_live_tokens(64)
                page = int(rng.choice([16, 16, 32, 64]))
                built = build(folder, dtype=dtype, kv_tokens=need, max_batch_tokens=max(need, 64), max_requests=8,
                              context=max(need, 512), page_size=page)
                got = run_plan_in_process(built.step_fn, plan)
                compare(plan, got, plain, *TOL[dtype], f"seed {seed} {cfg} page {page} {dtype}/{what}")
                assert built.cache.free_pages == built.cache.num_pages
