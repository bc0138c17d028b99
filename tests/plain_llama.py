"""A plain, slow Llama for tests: whole sequences, no cache, one function per part.

Written from the reference's formulas; every function cites the file and lines of
dynalm-project/dynalm it restates (paths are relative to that project's root). It shares
no code with `dynalm_b200`: it reads config.json and model.safetensors by itself and
computes in float64 with NumPy, except where the reference's 32-bit rounding is part of the
formula (rotary frequencies and angles).

tests/golden/ holds logits of the reference's own CPU `Transformer` on two tiny random
models; tests/test_plain_vs_reference.py checks this file against them.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# --------------------------------------------------------------------------------------------
# files
# --------------------------------------------------------------------------------------------

def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """u64 header length, JSON header, raw data
    (dynalm/src/loader/safetensors/safetensors.cpp:47-128). Returns float64 arrays."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        buf = data[b:en]
        if e["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            # bf16 is the upper half of an fp32 (dynacore/include/dynacore/tensor/fp16.h:18-73)
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            a = u.view(np.float32).astype(np.float64)
        elif e["dtype"] == "F16":
            a = np.frombuffer(buf, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"dtype {e['dtype']} of {name}")
        out[name] = a.reshape(e["shape"])
    return out


def read_config(path: str) -> dict:
    """config.json with the reference's defaults filled in
    (dynalm/src/loader/hf/hf_model.cpp:158-256)."""
    with open(path) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    c.setdefault("num_key_value_heads", heads)                       # :180
    if c.get("num_key_value_heads") is None:
        c["num_key_value_heads"] = heads
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // heads                     # :181
    c.setdefault("max_position_embeddings", 2048)                    # :182
    c.setdefault("rms_norm_eps", 1e-6)                               # :189
    c.setdefault("rope_theta", 10000.0)                              # :196
    c.setdefault("partial_rotary_factor", 1.0)                       # :197
    c.setdefault("embedding_multiplier", 1.0)                        # :249
    c.setdefault("residual_multiplier", 1.0)                         # :250
    c.setdefault("attention_multiplier", 0.0)                        # :251
    c.setdefault("logits_scaling", 1.0)                              # :252
    return c


# --------------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------------

def embed(table: np.ndarray, tokens: Sequence[int], scale: float = 1.0) -> np.ndarray:
    """x[i,:] = table[tok_i,:], scaled only when the multiplier is not 1
    (dynalm/src/model/transformer.cpp:576-577; dynacore/cpu/cpu_device.cpp:212-219)."""
    x = table[np.asarray(tokens, dtype=np.int64)].astype(np.float64)
    return x * scale if scale != 1.0 else x


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """inv = 1/sqrt(mean(x^2) + eps); y = x * inv * w, eps as a 32-bit float
    (dynacore/cpu/cpu_device.cpp:1179-1205; eps cast at dynalm/src/loader/hf/hf_model.cpp:189)."""
    eps = float(np.float32(eps))
    ss = np.sum(x * x, axis=-1, keepdims=True)
    inv = 1.0 / np.sqrt(ss / x.shape[-1] + eps)
    return x * inv * weight


def llama3_factors(c: dict) -> Optional[np.ndarray]:
    """Per-pair divisors of the rotary frequencies for rope_type llama3
    (dynalm/src/loader/hf/hf_model.cpp:378-406). None when there is no such block."""
    rs = c.get("rope_scaling")
    if not rs:
        return None
    kind = rs.get("rope_type", rs.get("type"))
    if kind != "llama3":
        return None
    factor = rs.get("factor", 8.0)
    low = rs.get("low_freq_factor", 1.0)
    high = rs.get("high_freq_factor", 4.0)
    old = rs.get("original_max_position_embeddings", 8192.0)
    rot = int(round(c["head_dim"] * c["partial_rotary_factor"]))
    base = float(np.float32(c["rope_theta"]))
    low_wl, high_wl = old / low, old / high
    out = []
    for i in range(0, rot, 2):
        freq = 1.0 / base ** (i / rot)
        wl = 2.0 * math.pi / freq
        if wl < high_wl:
            f = 1.0
        elif wl > low_wl:
            f = factor
        else:
            smooth = (old / wl - low) / (high - low)
            f = 1.0 / ((1.0 - smooth) / factor + smooth)
        out.append(f)
    return np.asarray(out, dtype=np.float32)


def rope_inv_freq(c: dict) -> np.ndarray:
    """inv_freq_i = base^(-2i/rot) / factor_i, all in 32-bit floats
    (dynacore/cpu/cpu_device.cpp:1233-1239)."""
    rot = int(round(c["head_dim"] * c["partial_rotary_factor"]))
    half = rot // 2
    base = np.float32(c["rope_theta"])
    i = np.arange(half, dtype=np.float32)
    expo = (np.float32(-2.0) * i) / np.float32(rot)
    inv = np.power(base, expo, dtype=np.float32)
    f = llama3_factors(c)
    if f is not None:
        inv = (inv / f).astype(np.float32)
    return inv


def rope(x: np.ndarray, positions: np.ndarray, c: dict) -> np.ndarray:
    """Half-split rotation of pairs (i, i + rot/2) of each head by theta = pos * inv_freq_i,
    theta a 32-bit product (dynacore/cpu/cpu_device.cpp:1240-1260; half-split for Hugging
    Face weights, dynalm/src/model/arch_llama.cpp:29). x: [n, heads, head_dim]."""
    inv = rope_inv_freq(c)
    half = inv.shape[0]
    pos_scale = np.float32(1.0)
    rs = c.get("rope_scaling") or {}
    if rs.get("rope_type", rs.get("type")) == "linear":
        pos_scale = np.float32(1.0) / np.float32(rs.get("factor", 1.0))
    p = positions.astype(np.float32) * pos_scale
    theta = (p[:, None] * inv[None, :]).astype(np.float32).astype(np.float64)   # [n, half]
    cos, sin = np.cos(theta)[:, None, :], np.sin(theta)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = a * sin + b * cos
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int = 0) -> np.ndarray:
    """Causal grouped-query attention of a whole sequence.
    s_t = scale * q.k_t for t in [max(0, pos-window+1), pos], softmax, weighted sum of v;
    query head h reads KV head h // (heads / kv_heads)
    (dynacore/cpu/cpu_device.cpp:1309-1412, 1717-1776; scale at
    dynalm/src/model/transformer.cpp:560). q: [n, heads, hd], k, v: [n, kv_heads, hd]."""
    n, heads, hd = q.shape
    group = heads // k.shape[1]
    out = np.zeros_like(q)
    for h in range(heads):
        kh, vh = k[:, h // group, :], v[:, h // group, :]
        s = scale * (q[:, h, :] @ kh.T)                                   # [n, n]
        pos = np.arange(n)
        mask = pos[None, :] > pos[:, None]
        if window > 0:
            mask |= pos[None, :] < pos[:, None] - window + 1
        s = np.where(mask, -np.inf, s)
        w = np.exp(s - s.max(axis=-1, keepdims=True))
        out[:, h, :] = (w @ vh) / w.sum(axis=-1, keepdims=True)
    return out


def silu(x: np.ndarray) -> np.ndarray:
    """x * sigmoid(x) (dynacore/cpu/cpu_device.cpp:117-123)."""
    return x / (1.0 + np.exp(-x))


def gated_mlp(x: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    """down(silu(gate x) * up x) (dynalm/src/model/transformer.cpp:671-693)."""
    return (silu(x @ gate.T) * (x @ up.T)) @ down.T


def attention_block(x: np.ndarray, w: Dict[str, np.ndarray], p: str, c: dict, positions: np.ndarray,
                    window: int = 0) -> np.ndarray:
    """q, k, v projections (+ bias when the tensor exists), RoPE on q and k, attention,
    output projection (dynalm/src/model/transformer.cpp:607-654)."""
    n = x.shape[0]
    heads, kvh, hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]

    def lin(name):
        y = x @ w[p + name + ".weight"].T
        b = w.get(p + name + ".bias")
        return y + b if b is not None else y

    q = lin("self_attn.q_proj").reshape(n, heads, hd)
    k = lin("self_attn.k_proj").reshape(n, kvh, hd)
    v = lin("self_attn.v_proj").reshape(n, kvh, hd)
    q, k = rope(q, positions, c), rope(k, positions, c)
    scale = c["attention_multiplier"] if c["attention_multiplier"] > 0 else 1.0 / math.sqrt(hd)
    scale = float(np.float32(scale))
    a = attention(q, k, v, scale, window).reshape(n, heads * hd)
    o = a @ w[p + "self_attn.o_proj.weight"].T
    b = w.get(p + "self_attn.o_proj.bias")
    return o + b if b is not None else o


def forward(c: dict, w: Dict[str, np.ndarray], tokens: Sequence[int], rows: Optional[Sequence[int]] = None) -> np.ndarray:
    """Logits [n, vocab] of a whole sequence from position 0 (with `rows`: at those positions only, as the
    reference gathers the wanted rows before the final norm, dynalm/src/model/transformer.cpp:703-718)
    (dynalm/src/model/transformer.cpp:498-733): embed; per layer x += attn(norm(x)),
    x += mlp(norm(x)), each scaled by the residual multiplier when it is not 1 (:656,:696);
    final norm; lm_head (the embedding table when the file has no lm_head,
    dynalm/src/model/arch_llama.cpp:32); logits divided by logits_scaling (:719)."""
    positions = np.arange(len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens, float(np.float32(c["embedding_multiplier"])))
    rscale = float(np.float32(c["residual_multiplier"]))
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = rms_norm(x, w[p + "input_layernorm.weight"], c["rms_norm_eps"])
        x = x + rscale * attention_block(h, w, p, c, positions)
        h = rms_norm(x, w[p + "post_attention_layernorm.weight"], c["rms_norm_eps"])
        x = x + rscale * gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                   w[p + "mlp.down_proj.weight"])
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    x = rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"])
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    logits = x @ head.T
    if c["logits_scaling"] != 1.0:
        logits = logits * float(np.float32(1.0) / np.float32(c["logits_scaling"]))
    return logits


class PlainLlama:
    """A model folder read for the plain implementation."""

    def __init__(self, folder: str):
        self.config = read_config(os.path.join(folder, "config.json"))
        self.weights = read_safetensors(os.path.join(folder, "model.safetensors"))

    def logits(self, tokens: Sequence[int], rows: Optional[Sequence[int]] = None) -> np.ndarray:
        return forward(self.config, self.weights, tokens, rows)

    def greedy(self, prompt: Sequence[int], steps: int) -> List[int]:
        """Whole-sequence recompute per new token; ties go to the lowest id
        (dynalm/src/sampling/sampler.cpp:31-38)."""
        seq = list(prompt)
        out = []
        for _ in range(steps):
            nxt = int(np.argmax(self.logits(seq)[-1]))
            out.append(nxt)
            seq.append(nxt)
        return out


# --------------------------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------------------------

_M64 = (1 << 64) - 1


class Xoshiro256:
    """xoshiro256** seeded through splitmix64; uniform = (next >> 11) * 2^-53
    (dynalm/src/sampling/sampler.cpp:55-81)."""

    def __init__(self, seed: int):
        x = seed & _M64
        self.s = []
        for _ in range(4):
            x = (x + 0x9E3779B97F4A7C15) & _M64
            z = x
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(x, k):
        return ((x << k) | (x >> (64 - k))) & _M64

    def next(self) -> int:
        s = self.s
        result = (self._rotl((s[1] * 5) & _M64, 7) * 9) & _M64
        t = (s[1] << 17) & _M64
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return result

    def uniform(self) -> float:
        return (self.next() >> 11) * 2.0 ** -53


def sample_temperature(logits: np.ndarray, temperature: float, u: float) -> int:
    """p_i = exp((l_i - max)/T); walk ids in order subtracting p_i from u * total until it
    goes negative; the last id on rounding (dynalm/src/sampling/sampler.cpp:120-137,209-220)."""
    l = logits.astype(np.float64)
    p = np.exp((l - l.max()) / temperature)
    r = u * p.sum()
    for i in range(len(p)):
        r -= p[i]
        if r < 0:
            return i
    return len(p) - 1
