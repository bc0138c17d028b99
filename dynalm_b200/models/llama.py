"""The Llama architecture: config.json -> LlamaConfig -> ModelPlan.

Tensor names are the Hugging Face ones the reference maps
(dynalm/src/loader/hf/hf_model.cpp:48-83). The block order (norm, attention, add, norm,
gated MLP, add) is `Transformer::forward_batch` for the Llama adapter
(dynalm/src/model/transformer.cpp:582-697, dynalm/src/model/arch_llama.cpp:23-39).
"""

from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Tuple

from ..config.llama import LLAMA_MODEL_TYPES, LlamaConfig
from ..config.plan import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec,
                           ModelPlan, NormSpec, PositionSpec)
from ..registry import register_architecture


def llama3_rope_factors(cfg: LlamaConfig) -> Optional[Tuple[float, ...]]:
    """Per-pair divisors of the rotary frequencies for rope_type "llama3".

    dynalm/src/loader/hf/hf_model.cpp:378-406: computed in double, one per pair
    (even i), stored as 32-bit floats.
    """
    rs = cfg.rope_scaling
    if rs is None or rs.rope_type != "llama3":
        return None
    import numpy as np

    rot = cfg.rotary_dim
    base = float(np.float32(cfg.rope_theta))
    low_wavelen = rs.original_max_position_embeddings / rs.low_freq_factor
    high_wavelen = rs.original_max_position_embeddings / rs.high_freq_factor
    out = []
    for i in range(0, rot, 2):
        freq = 1.0 / math.pow(base, i / rot)
        wavelen = 2.0 * math.pi / freq
        if wavelen < high_wavelen:
            f = 1.0
        elif wavelen > low_wavelen:
            f = rs.factor
        else:
            smooth = (rs.original_max_position_embeddings / wavelen - rs.low_freq_factor) / (
                rs.high_freq_factor - rs.low_freq_factor)
            f = 1.0 / ((1.0 - smooth) / rs.factor + smooth)
        out.append(float(np.float32(f)))
    return tuple(out)


class LlamaArchitecture:
    name = "LlamaForCausalLM"
    model_types = LLAMA_MODEL_TYPES

    def read_config(self, obj: Mapping[str, Any]) -> LlamaConfig:
        return LlamaConfig.from_dict(obj)

    def plan(self, cfg: LlamaConfig, present: Optional[set] = None) -> ModelPlan:
        """`present`: names of the tensors in the model folder, when known. Optional tensors
        (biases, lm_head) are decided by presence as the reference's adapter does
        (dynalm/src/model/arch_llama.cpp:30-32)."""
        has = (lambda n: n in present) if present is not None else (lambda n: False)
        rs = cfg.rope_scaling
        position = PositionSpec(
            kind="rotary",
            head_dim=cfg.head_dim,
            rotary_dim=cfg.rotary_dim,
            theta=cfg.rope_theta,
            pos_scale=(1.0 / rs.factor) if (rs is not None and rs.rope_type == "linear") else 1.0,
            factors=llama3_rope_factors(cfg),
        )
        layers = []
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}."
            mixer_tensors = {
                "q": p + "self_attn.q_proj.weight",
                "k": p + "self_attn.k_proj.weight",
                "v": p + "self_attn.v_proj.weight",
                "o": p + "self_attn.o_proj.weight",
            }
            for local, name in (("q_bias", "self_attn.q_proj.bias"), ("k_bias", "self_attn.k_proj.bias"),
                                ("v_bias", "self_attn.v_proj.bias"), ("o_bias", "self_attn.o_proj.bias")):
                if has(p + name):
                    mixer_tensors[local] = p + name
            layers.append(BlockSpec(
                "pre_norm",
                mixer_norm=NormSpec("rms", cfg.hidden_size, cfg.rms_norm_eps,
                                    {"weight": p + "input_layernorm.weight"}),
                mixer=MixerSpec(
                    "attention", cfg.hidden_size, mixer_tensors, num_heads=cfg.num_attention_heads,
                    num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                    scale=cfg.attention_scale, window=0, position=position),
                ffn_norm=NormSpec("rms", cfg.hidden_size, cfg.rms_norm_eps,
                                  {"weight": p + "post_attention_layernorm.weight"}),
                ffn=FeedForwardSpec(
                    "gated_mlp", cfg.hidden_size,
                    {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                     "down": p + "mlp.down_proj.weight"}, inner=cfg.intermediate_size, activation="silu"),
                residual_scale=cfg.residual_multiplier,
            ))
        # Tied unless the file carries lm_head.weight (arch_llama.cpp:32); without a file
        # listing, the declared key decides.
        tied = (not has("lm_head.weight")) if present is not None else cfg.tie_word_embeddings
        plan = ModelPlan(
            embedding=EmbeddingSpec(cfg.vocab_size, cfg.hidden_size, cfg.embedding_multiplier,
                                    {"weight": "model.embed_tokens.weight"}),
            layers=layers,
            order=[LayerRun(l) for l in range(cfg.num_hidden_layers)],
            final_norm=NormSpec("rms", cfg.hidden_size, cfg.rms_norm_eps, {"weight": "model.norm.weight"}),
            head=HeadSpec(cfg.vocab_size, cfg.hidden_size, tied, cfg.logits_scaling,
                          {} if tied else {"weight": "lm_head.weight"}),
            context_length=cfg.max_position_embeddings,
            # buffers that older Hugging Face checkpoints carry and nothing reads
            ignorable=tuple(f"model.layers.{l}.self_attn.rotary_emb.inv_freq" for l in range(cfg.num_hidden_layers)),
        )
        plan.validate()
        return plan


register_architecture(LlamaArchitecture())
