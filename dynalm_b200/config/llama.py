"""LlamaConfig: the keys of a Llama config.json, typed, with the reference's defaults.

Key names, defaults and refusals follow `hf::read_config`
(dynalm/src/loader/hf/hf_model.cpp:158-256), the llama3 block follows
`llama3_rope_factors` (:378-406), structural checks follow `ModelConfig::validate`
and `check_limits` (dynalm/src/model_ir/model_config.cpp:14-72) and the Llama
adapter (dynalm/src/model/arch_llama.cpp:23-39).
"""

from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from ..errors import Corrupt, InvalidArgument, Unsupported
from .reader import KeyReader

# model_type values the reference routes to its "llama" adapter
# (dynalm/src/loader/hf/hf_model.cpp:164).
LLAMA_MODEL_TYPES = ("llama", "mistral", "mixtral")

# Upper bounds on sizes read from an untrusted file
# (dynalm/src/model_ir/model_config.cpp:24-30).
_LIMITS = {
    "num_hidden_layers": 1024,
    "hidden_size": 1 << 17,
    "intermediate_size": 1 << 19,
    "num_attention_heads": 1024,
    "num_key_value_heads": 1024,
    "head_dim": 4096,
    "vocab_size": 1 << 24,
    "max_position_embeddings": 1 << 24,
}


@dataclass(frozen=True)
class RopeScaling:
    """The `rope_scaling` object. `rope_type` is "default", "linear" or "llama3"."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: float = 8192.0

    def to_dict(self) -> dict:
        if self.rope_type == "llama3":
            return {
                "rope_type": "llama3",
                "factor": self.factor,
                "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings,
            }
        return {"rope_type": self.rope_type, "factor": self.factor}


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = True
    # Multipliers the reference reads for every model_type (hf_model.cpp:249-253).
    embedding_multiplier: float = 1.0
    residual_multiplier: float = 1.0
    attention_multiplier: float = 0.0  # 0 means 1/sqrt(head_dim) (transformer.cpp:560)
    logits_scaling: float = 1.0
    model_type: str = "llama"

    architecture_name = "LlamaForCausalLM"

    # ---- derived sizes -------------------------------------------------------------------
    @property
    def rotary_dim(self) -> int:
        # hf_model.cpp:197: lround(head_dim * partial_rotary_factor), halves away from zero
        return int(math.floor(self.head_dim * self.partial_rotary_factor + 0.5))

    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def attention_scale(self) -> float:
        return self.attention_multiplier if self.attention_multiplier > 0 else self.head_dim ** -0.5

    def kv_bytes_per_token(self, elem_bytes: int) -> int:
        # model_config.cpp:9-12
        return 2 * self.kv_width * self.num_hidden_layers * elem_bytes

    # ---- reading -------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, obj: Mapping[str, Any]) -> "LlamaConfig":
        r = KeyReader(obj)
        model_type = r.str_or("model_type", None)
        if model_type is None:
            raise Corrupt("config.json: missing model_type")
        if model_type not in LLAMA_MODEL_TYPES:
            raise Unsupported(f"config.json: model_type '{model_type}' is not a Llama-family type "
                              f"(supported: {', '.join(LLAMA_MODEL_TYPES)})")
        vocab = r.int("vocab_size")
        hidden = r.int("hidden_size")
        inter = r.int("intermediate_size")
        layers = r.int("num_hidden_layers")
        heads = r.int("num_attention_heads")
        if heads <= 0 or layers <= 0:
            raise Corrupt("config.json: layer and head counts must be > 0")
        kv_heads = r.int_or("num_key_value_heads", heads)
        head_dim = r.int_or("head_dim", hidden // heads)
        if r.int_or("num_local_experts", 0) > 0:
            raise Unsupported("config.json: expert (MoE) feed-forward layers are not built in this engine")
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            if r.float_or(key, 0.0) != 0.0:
                raise Unsupported(f"config.json: '{key}' is not supported")

        scaling = None
        rs = r.object_or_none("rope_scaling")
        if rs is not None:
            kind = rs.str_or("rope_type", None) or rs.str_or("type", None) or ""
            if kind == "linear":
                scaling = RopeScaling("linear", factor=rs.float_or("factor", 1.0))
            elif kind == "llama3":
                scaling = RopeScaling(
                    "llama3",
                    factor=rs.float_or("factor", 8.0),
                    low_freq_factor=rs.float_or("low_freq_factor", 1.0),
                    high_freq_factor=rs.float_or("high_freq_factor", 4.0),
                    original_max_position_embeddings=rs.float_or("original_max_position_embeddings", 8192.0),
                )
            elif kind == "yarn":
                # arch_llama.cpp:33-35
                raise Unsupported("Llama with YaRN RoPE scaling is not supported yet")
            elif kind not in ("", "default"):
                raise Unsupported(f"rope_scaling type '{kind}' is not supported yet")

        cfg = cls(
            vocab_size=vocab,
            hidden_size=hidden,
            intermediate_size=inter,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=r.int_or("max_position_embeddings", 2048),
            rms_norm_eps=r.float_or("rms_norm_eps", 1e-6),
            rope_theta=r.float_or("rope_theta", 10000.0),
            partial_rotary_factor=r.float_or("partial_rotary_factor", 1.0),
            rope_scaling=scaling,
            # Declared intent; the loader overrides it from the presence of lm_head.weight
            # as the reference's adapter does (arch_llama.cpp:32).
            tie_word_embeddings=r.bool_or("tie_word_embeddings", True),
            embedding_multiplier=r.float_or("embedding_multiplier", 1.0),
            residual_multiplier=r.float_or("residual_multiplier", 1.0),
            attention_multiplier=r.float_or("attention_multiplier", 0.0),
            logits_scaling=r.float_or("logits_scaling", 1.0),
            model_type=model_type,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        def bad(msg: str):
            raise InvalidArgument("model config: " + msg)

        for name, limit in _LIMITS.items():
            value = getattr(self, name)
            if value > limit:
                bad(f"{name} {value} exceeds the supported maximum {limit}")
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                bad(f"{name} must be > 0")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            bad(f"num_heads ({self.num_attention_heads}) not divisible by num_kv_heads "
                f"({self.num_key_value_heads})")
        rot = self.rotary_dim
        if rot <= 0 or rot > self.head_dim or rot % 2 != 0:
            bad(f"rope dim {rot} invalid for head_dim {self.head_dim}")
        if not self.rope_theta > 0:
            bad("rope freq_base must be > 0")
        if not self.rms_norm_eps > 0:
            bad("norm_eps must be > 0")
        if not self.logits_scaling > 0:
            bad("logits_scaling must be > 0")
        rs = self.rope_scaling
        if rs is not None and rs.rope_type == "llama3":
            if rs.factor <= 0 or rs.high_freq_factor <= rs.low_freq_factor or rs.original_max_position_embeddings <= 0:
                raise Corrupt("config.json: invalid llama3 rope_scaling")
        if rs is not None and rs.rope_type == "linear" and not rs.factor > 0:
            raise Corrupt("config.json: invalid linear rope_scaling")

    # ---- writing -------------------------------------------------------------------------
    def to_dict(self) -> dict:
        out = {
            "architectures": [self.architecture_name],
            "model_type": self.model_type,
        }
        for f in dataclasses.fields(self):
            if f.name in ("rope_scaling", "model_type"):
                continue
            out[f.name] = getattr(self, f.name)
        out["rope_scaling"] = self.rope_scaling.to_dict() if self.rope_scaling else None
        out["hidden_act"] = "silu"
        out["torch_dtype"] = "bfloat16"
        return out

    def with_tied(self, tied: bool) -> "LlamaConfig":
        return dataclasses.replace(self, tie_word_embeddings=tied)
