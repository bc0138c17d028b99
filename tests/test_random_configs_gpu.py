"""Replay on the GPU for configurations drawn at random (seeded): head counts and groups, head sizes in steps of 16
and widths, inner widths and vocabularies of any size, one to three layers, every kind of rotary scaling the
architecture reads, tied and untied heads, with and without attention biases. Each is replayed in portions of
changing size and mixed with reused pages, in 32-bit and in bfloat16, against the plain implementation, with the
tolerances of test_replay_gpu.py. The fixed tiny configurations pin the options one by one; this pins their
combinations."""

import numpy as np
import pytest

from plain_llama import PlainLlama
from replay_util import compare, kl_and_top1, plan_chunks, plan_mixed, random_requests, run_plan_in_process
from test_replay_gpu import KL_GATE, NEAR_TIE, SIZES, TOL

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    """(config.json dict, optional tensor names) from a seed."""
    rng = np.random.RandomState(1000 + seed)
    kv = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 5]))
    heads = kv * group
    head_dim = int(rng.choice([16, 32, 48, 64, 80, 96, 112, 128]))
    layers = int(rng.randint(1, 4))
    hidden = int(rng.choice([40, 56, 64, 72, 88, 100, 120, 136]))
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": int(rng.randint(60, 700)), "hidden_size": hidden,
        "intermediate_size": int(rng.choice([8, 4, 1])) * int(rng.randint(9, 30)), "num_hidden_layers": layers,
        "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": head_dim,
        "max_position_embeddings": 512, "rms_norm_eps": float(10.0 ** rng.uniform(-6.5, -4.5)),
        "rope_theta": float(rng.choice([10000.0, 25000.0, 500000.0, 1000000.0])),
        "tie_word_embeddings": bool(rng.randint(2)),
    }
    scaling = rng.randint(3)
    if scaling == 1:
        cfg["rope_scaling"] = {"rope_type": "llama3", "factor": float(rng.choice([4.0, 8.0, 32.0])), "low_freq_factor": 1.0,
                               "high_freq_factor": 4.0, "original_max_position_embeddings": int(rng.choice([32, 64, 128]))}
    elif scaling == 2:
        cfg["rope_scaling"] = {"type": "linear", "factor": float(rng.choice([2.0, 4.0]))}
    if rng.randint(3) == 0:
        cfg["partial_rotary_factor"] = 0.5
    optional = []
    if rng.randint(3) == 0:
        optional = [f"model.layers.{l}.self_attn.{p}_proj.bias" for l in range(layers) for p in "qkvo"]
    return cfg, optional


@pytest.mark.parametrize("seed", range(12))
def test_a_configuration_drawn_at_random(seed, tmp_path):
    import torch
    from dynalm_b200.engine import build
    from dynalm_b200.weights import write_model_folder
    cfg, optional = draw_config(seed)
    rng = np.random.RandomState(seed)
    lengths = [int(n) for n in rng.randint(1, 200, size=5)] + [int(rng.choice([64, 128, 129]))]
    reqs = random_requests(cfg["vocab_size"], lengths, seed=200 + seed)
    for dtype, torch_dtype in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder = str(tmp_path / dtype)
        write_model_folder(folder, cfg, 50 + seed, dtype=torch_dtype, optional=optional or None)
        model = PlainLlama(folder)
        plain = {r: model.logits(t) for r, t in reqs.items()}
        for what, plan in (("chunks", plan_chunks(reqs, SIZES)), ("mixed", plan_mixed(reqs, seed=seed, max_live=4))):
            need = plan.max_live_tokens(64)
            built = build(folder, dtype=dtype, kv_tokens=need, max_batch_tokens=max(need, 64), max_requests=8,
                          context=max(need, 256))
            got = run_plan_in_process(built.step_fn, plan)
            label = f"seed {seed} {cfg['num_attention_heads']}:{cfg['num_key_value_heads']} heads of {cfg['head_dim']}, width " \
                    f"{cfg['hidden_size']}, {dtype}, {what}"
            worst = compare(plan, got, plain, TOL[dtype][0], TOL[dtype][1], label)
            assert built.cache.free_pages == built.cache.num_pages, "pages were lost"
            kl, top1 = kl_and_top1(plan, got, plain, near_tie=NEAR_TIE[dtype])
            print(f"{label}: worst {worst:.3g} KL {kl:.3g} top-1 {top1:.4f}")
            assert kl <= KL_GATE[dtype] and top1 == 1.0, f"{label}: mean KL {kl:.3g}, top-1 agreement {top1:.4f}"
