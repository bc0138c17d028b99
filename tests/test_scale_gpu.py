"""The Llama 3.2 1B layer sizes (4 of its 16 layers, the full vocabulary, tied embeddings, llama3 RoPE
scaling) with random weights: the float32 engine gives equal logits however the prompt is cut, and the
bfloat16 engine (tcgen05 products, flash attention, the decode kernels and graphs) agrees with it the
way the reference asks of its own GPU path: mean KL at most 0.0025 and nearly all top-1 tokens equal
(dynalm/benchmarks/bench_gpu_accuracy.cpp:91-92)."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 4, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}


@pytest.fixture(scope="module")
def tensors():
    from dynalm_b200.registry import find_architecture
    from dynalm_b200.weights import random_tensors
    arch = find_architecture(CFG)
    t = random_tensors(arch.plan(arch.read_config(CFG)), 0, torch.bfloat16)
    # random N(0, 0.02) weights give nearly flat logits; a wider embedding makes the distribution peaked
    # enough for top-1 and KL to mean something
    t["model.embed_tokens.weight"] = (t["model.embed_tokens.weight"].float() * 8).to(torch.bfloat16)
    return t


def _logits(tensors, dtype, cuts, tokens, want_from):
    from dynalm_b200 import StepEntry
    from dynalm_b200.engine import build
    built = build(config_obj=CFG, tensors=tensors, dtype=dtype, kv_tokens=1024, max_batch_tokens=512, max_requests=4)
    out, pos = [], 0
    for c in cuts:
        want = [i for i in range(c) if pos + i >= want_from]
        got = built.step_fn.step([StepEntry("r", tokens[pos:pos + c], want)])
        if got is not None:
            out.append(got.float().cpu().numpy().copy())
        pos += c
    built.step_fn.end("r")
    del built
    torch.cuda.empty_cache()
    return np.concatenate(out)


def test_one_b_shape_parity(tensors):
    rng = np.random.RandomState(0)
    tokens = [int(t) for t in rng.randint(0, CFG["vocab_size"], 400)]
    want_from = 336                                    # the last 64 positions
    whole32 = _logits(tensors, "float32", [400], tokens, want_from)
    cut32 = _logits(tensors, "float32", [300, 37, 2, 29] + [1] * 32, tokens, want_from)
    assert np.abs(whole32 - cut32).max() <= 1e-4 * max(1.0, np.abs(whole32).max())
    for cuts in ([400], [300, 37, 2, 29] + [1] * 32):
        got = _logits(tensors, "bfloat16", cuts, tokens, want_from)
        ref = whole32.astype(np.float64)
        lp_ref = ref - np.log(np.exp(ref - ref.max(-1, keepdims=True)).sum(-1, keepdims=True)) - ref.max(-1, keepdims=True)
        g = got.astype(np.float64)
        lp_got = g - np.log(np.exp(g - g.max(-1, keepdims=True)).sum(-1, keepdims=True)) - g.max(-1, keepdims=True)
        kl = (np.exp(lp_ref) * (lp_ref - lp_got)).sum(-1).mean()
        top1 = (ref.argmax(-1) == g.argmax(-1)).mean()
        print(f"cuts {len(cuts)}: mean KL {kl:.2e}, top-1 agreement {top1:.3f}")
        assert kl <= 0.0025 and top1 >= 0.9
