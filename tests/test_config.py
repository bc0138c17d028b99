"""Configuration and registry: keys, defaults, refusals."""

import copy

import pytest

import dynalm_b200
from dynalm_b200.config import LlamaConfig
from dynalm_b200.errors import Corrupt, InvalidArgument, NotFound, Unsupported
from dynalm_b200.models.llama import llama3_rope_factors
from dynalm_b200.registry import find_architecture, registered_architectures
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_defaults_follow_the_reference():
    c = LlamaConfig.from_dict({"model_type": "llama", "vocab_size": 100, "hidden_size": 64, "intermediate_size": 128,
                               "num_hidden_layers": 2, "num_attention_heads": 4})
    assert c.num_key_value_heads == 4 and c.head_dim == 16
    assert c.max_position_embeddings == 2048 and c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.tie_word_embeddings is True and c.rope_scaling is None
    assert c.attention_scale == 16 ** -0.5 and c.rotary_dim == 16


def test_explicit_head_dim_and_llama3_block():
    c = LlamaConfig.from_dict(TINY_B)
    assert c.head_dim == 32 and c.q_width == 192 != c.hidden_size
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.original_max_position_embeddings == 32
    f = llama3_rope_factors(c)
    # the values the reference's own loader computes for this block (rope_freqs 1.0000 2.0514 8.0000 ...)
    assert len(f) == 16 and f[0] == 1.0 and abs(f[1] - 2.0514) < 1e-4 and all(x == 8.0 for x in f[2:])


def test_multipliers_and_partial_rotary():
    c = LlamaConfig.from_dict(TINY_C)
    assert c.rotary_dim == 24 and c.attention_scale == 0.2 and c.logits_scaling == 4.0
    assert c.rope_scaling.rope_type == "linear" and c.rope_scaling.factor == 2.0
    plan = find_architecture(TINY_C).plan(c)
    assert plan.layers[0].mixer.position.pos_scale == 0.5 and plan.layers[0].residual_scale == 0.5
    assert plan.embedding.scale == 3.0 and plan.head.logit_divisor == 4.0


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads"])
def test_missing_key(key):
    d = copy.deepcopy(TINY_A)
    del d[key]
    with pytest.raises(NotFound, match=f"missing '{key}'"):
        LlamaConfig.from_dict(d)


def test_refusals():
    def mod(**kw):
        d = copy.deepcopy(TINY_B)
        d.update(kw)
        return d
    with pytest.raises(Corrupt):
        LlamaConfig.from_dict(mod(hidden_size="96"))
    with pytest.raises(Corrupt):
        LlamaConfig.from_dict(mod(hidden_size=96.5))
    with pytest.raises(InvalidArgument, match="not divisible"):
        LlamaConfig.from_dict(mod(num_key_value_heads=4))
    with pytest.raises(InvalidArgument, match="exceeds the supported maximum"):
        LlamaConfig.from_dict(mod(vocab_size=1 << 25))
    with pytest.raises(Unsupported, match="YaRN"):
        LlamaConfig.from_dict(mod(rope_scaling={"rope_type": "yarn", "factor": 4.0}))
    with pytest.raises(Unsupported, match="dynamic"):
        LlamaConfig.from_dict(mod(rope_scaling={"rope_type": "dynamic", "factor": 4.0}))
    with pytest.raises(Corrupt, match="invalid llama3"):
        LlamaConfig.from_dict(mod(rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 4.0,
                                                "high_freq_factor": 1.0}))
    with pytest.raises(Unsupported, match="MoE"):
        LlamaConfig.from_dict(mod(num_local_experts=8))
    with pytest.raises(Corrupt, match="model_type"):
        LlamaConfig.from_dict({k: v for k, v in TINY_A.items() if k != "model_type"})
    with pytest.raises(InvalidArgument, match="rope dim"):
        LlamaConfig.from_dict(mod(partial_rotary_factor=0.03))


def test_registry():
    assert "LlamaForCausalLM" in registered_architectures()
    assert find_architecture(TINY_A).name == "LlamaForCausalLM"
    assert find_architecture({"model_type": "mistral"}).name == "LlamaForCausalLM"     # fallback on model_type
    with pytest.raises(Unsupported, match="registered: .*LlamaForCausalLM"):
        find_architecture({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"})
    with pytest.raises(Unsupported):
        find_architecture({"model_type": "gemma"})


def test_plan_is_data():
    arch = find_architecture(TINY_B)
    plan = arch.plan(arch.read_config(TINY_B), present={"lm_head.weight"})
    assert len(plan.layers) == 3 and [r.layer for r in plan.order] == [0, 1, 2]
    assert not plan.head.tied
    assert arch.plan(arch.read_config(TINY_B), present=set()).head.tied      # tied when the file has no lm_head
    m = plan.layers[1].mixer
    assert (m.kind, m.num_heads, m.num_kv_heads, m.head_dim, m.window) == ("attention", 6, 2, 32, 0)
    assert m.tensors["q"] == "model.layers.1.self_attn.q_proj.weight"
    # a plan that names a layer twice and lets an entry read another's cache is valid data
    from dynalm_b200.config import LayerRun
    plan.order = [LayerRun(0), LayerRun(1), LayerRun(1, cache_of=1), LayerRun(2)]
    plan.validate()
    plan.order = [LayerRun(0, cache_of=1), LayerRun(1)]
    with pytest.raises(InvalidArgument, match="not earlier"):
        plan.validate()


def test_round_trip_to_dict():
    c = LlamaConfig.from_dict(TINY_B)
    assert LlamaConfig.from_dict(c.to_dict()) == c
