"""Each part alone against the plain function of the same part, and a toy mixer with state of its
own that is registered, built and stepped without touching the framework."""

import os

import numpy as np
import pytest
import torch

import plain_llama as plain
from tiny_configs import TINY_B, TINY_C

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def _runtime(dtype, max_tokens=256):
    from dynalm_b200.engine import Runtime
    return Runtime(DEV, dtype, max_tokens)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from dynalm_b200.config import NormSpec
    from dynalm_b200.parts import NORMS
    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.1 * torch.randn(96, generator=g)
    x = torch.randn(11, 96, generator=g) * 2
    part = NORMS.get("rms")(NormSpec("rms", 96, 1e-6), {"weight": w.to(DEV)}, rt)
    out = torch.empty(11, 96, dtype=dtype, device=DEV)
    part.forward(x.to(DEV), out)
    ref = plain.rms_norm(x.double().numpy(), w.double().numpy(), 1e-6)
    assert np.abs(out.float().cpu().numpy() - ref).max() <= _tol(dtype) * 4


def test_rotary_part_frequencies():
    from dynalm_b200.parts import POSITIONS
    from dynalm_b200.registry import find_architecture
    rt = _runtime(torch.float32)
    for cfg in (TINY_B, TINY_C):
        arch = find_architecture(cfg)
        spec = arch.plan(arch.read_config(cfg)).layers[0].mixer.position
        part = POSITIONS.get(spec.kind)(spec, rt)
        inv, rot, scale = part.table()
        ref = plain.rope_inv_freq(plain.read_config_dict(cfg) if hasattr(plain, "read_config_dict") else _filled(cfg))
        assert rot == 2 * len(ref) and np.array_equal(inv.cpu().numpy(), ref)


def _filled(cfg):
    c = dict(cfg)
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("partial_rotary_factor", 1.0)
    c.setdefault("rope_theta", 10000.0)
    return c


def _context(rt, cache, entries, vocab=1000):
    from dynalm_b200.engine import BatchBuilder, StepEntry
    b = BatchBuilder(cache, rt, 8, vocab)
    return b, b.build([StepEntry(r, t, []) for r, t in entries])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixer_alone(dtype):
    """The mixer over two requests cut into portions equals the plain attention block on whole sequences."""
    from dynalm_b200.cache import CacheManager
    from dynalm_b200.engine import BatchBuilder, StepEntry
    from dynalm_b200.parts import MIXERS
    from dynalm_b200.registry import find_architecture
    cfg = plain_cfg = _filled(dict(TINY_B, attention_multiplier=0.0, residual_multiplier=1.0))
    arch = find_architecture(TINY_B)
    spec = arch.plan(arch.read_config(TINY_B)).layers[0].mixer
    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(1)
    H, qw, kw = 96, 192, 64
    t = {"q": torch.randn(qw, H, generator=g) * 0.1, "k": torch.randn(kw, H, generator=g) * 0.1,
         "v": torch.randn(kw, H, generator=g) * 0.1, "o": torch.randn(H, qw, generator=g) * 0.1}
    mixer = MIXERS.get("attention")(spec, {n: v.to(DEV, dtype) for n, v in t.items()}, rt)
    cache = CacheManager([mixer.cache_spec()], 16, 256, 8, 256, DEV, dtype)
    builder = BatchBuilder(cache, rt, 8, 1000, mixer.step_plans())
    lens = {"a": 50, "b": 21}
    xs = {r: torch.randn(n, H, generator=g) for r, n in lens.items()}
    w = {"p.self_attn." + n + "_proj.weight": v.to(dtype).double().numpy() for n, v in t.items()}
    ref = {r: plain.attention_block(xs[r].to(dtype).double().numpy(), w, "p.", plain_cfg, np.arange(lens[r]))
           for r in lens}
    got = {r: [] for r in lens}
    cuts = [[("a", 0, 17), ("b", 0, 2)], [("b", 2, 19)], [("a", 17, 32), ("b", 21, 0)], [("a", 49, 1)]]
    for step in cuts:
        entries = [(r, s, n) for r, s, n in step if n > 0]
        ctx = builder.build([StepEntry(r, [0] * n, []) for r, s, n in entries])
        x = torch.cat([xs[r][s:s + n] for r, s, n in entries]).to(DEV, dtype)
        view = cache.view(0, builder.tables)
        y = mixer.forward(x, ctx, view, True).float().cpu()
        builder.finish([StepEntry(r, [0] * n, []) for r, s, n in entries])
        o = 0
        for r, s, n in entries:
            got[r].append(y[o:o + n])
            o += n
    for r in lens:
        err = np.abs(torch.cat(got[r]).numpy() - ref[r]).max()
        assert err <= _tol(dtype) * max(1.0, np.abs(ref[r]).max()), f"{r}: {err}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_alone(dtype):
    from dynalm_b200.config import FeedForwardSpec
    from dynalm_b200.parts import FEED_FORWARDS
    rt = _runtime(dtype)
    g = torch.Generator().manual_seed(2)
    W, F = 80, 112
    t = {"gate": torch.randn(F, W, generator=g) * 0.2, "up": torch.randn(F, W, generator=g) * 0.2,
         "down": torch.randn(W, F, generator=g) * 0.2}
    part = FEED_FORWARDS.get("gated_mlp")(FeedForwardSpec("gated_mlp", W, inner=F), {n: v.to(DEV, dtype) for n, v in t.items()}, rt)
    x = torch.randn(9, W, generator=g)
    y = part.forward(x.to(DEV, dtype), None).float().cpu().numpy()
    d = {n: v.to(dtype).double().numpy() for n, v in t.items()}
    ref = plain.gated_mlp(x.to(dtype).double().numpy(), d["gate"], d["up"], d["down"])
    assert np.abs(y - ref).max() <= _tol(dtype) * max(1.0, np.abs(ref).max())


# ---------------------------------------------------------------------------------------------
# a toy architecture defined here: one attention layer, then a layer whose mixer keeps a running
# state per request, run twice, the second time sharing nothing; plus an entry that reads another
# entry's cache
# ---------------------------------------------------------------------------------------------

def _register_toy():
    from dynalm_b200.config import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan,
                                    NormSpec, PositionSpec)
    from dynalm_b200.parts import CacheSpec, TensorDecl, register_mixer
    from dynalm_b200.registry import register_architecture

    @register_mixer("toy_decay")
    class ToyDecay:
        """y_t = W x_t + 0.5 * s_{t-1}; s_t = y_t. The state s is one row per request."""

        @staticmethod
        def declare(spec):
            return {"w": TensorDecl((spec.width, spec.width))}

        def __init__(self, spec, tensors, runtime):
            self.spec, self.w, self.rt = spec, tensors["w"], runtime

        def cache_spec(self):
            return CacheSpec(kind="state", state_shape=(self.spec.width,), dtype="float32")

        def forward(self, x, ctx, cache, owns_cache=True):
            state = cache.arrays[0]
            proj = (x.float() @ self.w.float().T)
            out = torch.empty_like(proj)
            r0 = 0
            for n, slot in zip(ctx.h_q_len, ctx.h_state_slots):
                s = state[slot].clone()
                for i in range(n):
                    s = proj[r0 + i] + 0.5 * s
                    out[r0 + i] = s
                state[slot] = s
                r0 += n
            return out.to(x.dtype)

    class ToyArch:
        name = "ToyForCausalLM"
        model_types = ("toy",)

        def read_config(self, obj):
            return dict(obj)

        def plan(self, c, present=None):
            W, V = c["width"], c["vocab"]

            def norm(n):
                return NormSpec("rms", W, 1e-5, {"weight": n})

            def ffn(p):
                return FeedForwardSpec("gated_mlp", W, {"gate": p + "gate", "up": p + "up", "down": p + "down"},
                                       inner=c["inner"], activation="silu")
            heads = dict(num_heads=c["heads"], num_kv_heads=c["kv_heads"], head_dim=c["head_dim"], scale=c["head_dim"] ** -0.5)
            attn = MixerSpec("attention", W, {"q": "l0.q", "k": "l0.k", "v": "l0.v", "o": "l0.o"}, window=0,
                             position=PositionSpec("rotary", c["head_dim"], c["head_dim"], 10000.0), **heads)
            win = MixerSpec("attention", W, {"q": "l2.q", "k": "l2.k", "v": "l2.v", "o": "l2.o"}, window=c["window"],
                            position=PositionSpec("none"), **heads)
            toy = MixerSpec("toy_decay", W, {"w": "l1.w"})

            def block(n, mixer):
                return BlockSpec("pre_norm", mixer_norm=norm(f"l{n}.n1"), mixer=mixer, ffn_norm=norm(f"l{n}.n2"),
                                 ffn=ffn(f"l{n}."))
            layers = [block(0, attn), block(1, toy), block(2, win)]
            # layer 1 is named twice; the last entry runs layer 0 again on the first entry's cache
            order = [LayerRun(0), LayerRun(1), LayerRun(2), LayerRun(1), LayerRun(0, cache_of=0)]
            return ModelPlan(EmbeddingSpec(V, W, 1.0, {"weight": "emb"}), layers, order, norm("final"),
                             HeadSpec(V, W, True), c["context"])

    register_architecture(ToyArch())
    return ToyArch


TOY = {"architectures": ["ToyForCausalLM"], "model_type": "toy", "width": 48, "vocab": 120, "inner": 64, "heads": 3,
       "kv_heads": 1, "head_dim": 16, "window": 24, "context": 256}


def _toy_reference(w, tokens):
    """Whole sequence, no cache, plain functions; mirrors ToyArch.plan."""
    c = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "partial_rotary_factor": 1.0,
         "rope_theta": 10000.0, "attention_multiplier": 0.0}
    n = len(tokens)
    x = w["emb"][np.asarray(tokens)]

    kept = {}

    def attn(h, p, rotary, window, read_cache_of=None):
        q = (h @ w[p + "q"].T).reshape(n, 3, 16)
        if rotary:
            q = plain.rope(q, np.arange(n), c)
        if read_cache_of is None:
            k = (h @ w[p + "k"].T).reshape(n, 1, 16)
            v = (h @ w[p + "v"].T).reshape(n, 1, 16)
            if rotary:
                k = plain.rope(k, np.arange(n), c)
            kept[p] = (k, v)
        else:
            k, v = kept[read_cache_of]       # the keys and values the earlier entry cached
        return plain.attention(q, k, v, 16 ** -0.5, window).reshape(n, 48) @ w[p + "o"].T

    def toy(h):
        proj = h @ w["l1.w"].T
        out = np.zeros_like(proj)
        s = np.zeros(48)
        for i in range(n):
            s = proj[i] + 0.5 * s
            out[i] = s
        return out

    def ffn(h, p):
        return plain.gated_mlp(h, w[p + "gate"], w[p + "up"], w[p + "down"])

    for p, mix in (("l0.", lambda h: attn(h, "l0.", True, 0)), ("l1.", toy), ("l2.", lambda h: attn(h, "l2.", False, 24)),
                   ("l1.", toy), ("l0.", lambda h: attn(h, "l0.", True, 0, read_cache_of="l0."))):
        x = x + mix(plain.rms_norm(x, w[p + "n1"], 1e-5))
        x = x + ffn(plain.rms_norm(x, w[p + "n2"], 1e-5), p)
    return plain.rms_norm(x, w["final"], 1e-5) @ w["emb"].T


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A model whose plan names a layer twice (each run with a state of its own), has a windowed
    attention layer beside a full one (two page groups) and an entry that reads another entry's
    cache. Whole requests and cut requests give the same logits, and both match plain functions."""
    _register_toy()
    from dynalm_b200.engine import StepEntry, build
    from dynalm_b200.weights import write_model_folder
    folder = str(tmp_path / "toy")
    write_model_folder(folder, TOY, 3, torch.float32)
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.RandomState(0)
    reqs = {"a": [int(t) for t in rng.randint(0, 120, 70)], "b": [int(t) for t in rng.randint(0, 120, 37)]}

    def run(cuts):
        built = build(folder, dtype="float32", kv_tokens=256, max_batch_tokens=128, max_requests=4)
        assert len(built.cache.groups) == 2                       # all keys | a window of them
        assert set(built.cache.state_arrays) == {1, 3}            # a state of its own per run of the toy layer
        out = {r: [] for r in reqs}
        pos = {r: 0 for r in reqs}
        for step in cuts:
            entries = []
            for r, n in step:
                entries.append(StepEntry(r, reqs[r][pos[r]:pos[r] + n], list(range(n))))
            logits = built.step_fn.step(entries).cpu().numpy()
            o = 0
            for r, n in step:
                out[r].append(logits[o:o + n].copy())
                pos[r] += n
                o += n
            built.cache.check()
        win_group = [g for g in built.cache.groups if g.spec.window > 0][0]
        assert win_group.pool.num_held < sum(-(-len(t) // 16) for t in reqs.values())   # the window gave pages back
        for r in reqs:
            built.step_fn.end(r)
        assert built.cache.free_pages == built.cache.num_pages
        return {r: np.concatenate(v) for r, v in out.items()}

    whole = run([[("a", 70)], [("b", 37)]])
    cut = run([[("a", 16), ("b", 5)], [("a", 7)], [("b", 2), ("a", 2)], [("a", 40), ("b", 29)], [("a", 1), ("b", 1)],
               [("a", 1)], [("a", 1)], [("a", 2)]])
    for r in reqs:
        ref = _toy_reference(w, reqs[r])
        assert np.abs(whole[r] - ref).max() <= 3e-5 * max(1.0, np.abs(ref).max()), f"{r}: whole vs plain"
        assert np.abs(cut[r] - ref).max() <= 3e-5 * max(1.0, np.abs(ref).max()), f"{r}: cut vs plain"


# ---------------------------------------------------------------------------------------------
# another arrangement of a layer, with a part of a kind of its own and parameters of its own, all defined here
# ---------------------------------------------------------------------------------------------

def test_toy_block_with_post_norms_and_a_third_part(tmp_path):
    """A block that nothing in the package knows: no norm before its parts but one after each (x = norm(x + part(x))),
    three parts instead of two (a mixer with a parameter of its own kind, `taps`; attention; a feed-forward), and a
    parameter of the arrangement (`skip`). It registers, loads, builds and steps without a change to the package, whole
    and cut, and matches the same arithmetic written out with NumPy."""
    from dynalm_b200.config import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan,
                                    NormSpec, PositionSpec)
    from dynalm_b200.engine import StepEntry, build
    from dynalm_b200.parts import TensorDecl, register_block, register_mixer
    from dynalm_b200.parts.base import build_part
    from dynalm_b200.registry import register_architecture
    from dynalm_b200.weights import write_model_folder
    W, V, HD = 32, 60, 16

    @register_mixer("toy_shift")
    class ShiftMix:
        """y[t] = x[t] W0 + x[t-1] W1 (+ x[t-2] W2 with taps = 3): the last taps-1 rows of a request are its state."""

        @staticmethod
        def declare(spec):
            return {f"w{i}": TensorDecl((spec.width, spec.width)) for i in range(spec.taps)}

        def __init__(self, spec, tensors, runtime):
            self.spec, self.w = spec, [tensors[f"w{i}"].float() for i in range(spec.taps)]

        def cache_spec(self):
            from dynalm_b200.parts import CacheSpec
            return CacheSpec(kind="state", state_shape=(self.spec.taps - 1, self.spec.width), dtype="float32")

        def forward(self, x, ctx, cache, owns_cache=True):
            state = cache.arrays[0]
            out = torch.empty_like(x, dtype=torch.float32)
            r0 = 0
            for n, slot in zip(ctx.h_q_len, ctx.h_state_slots):
                rows = torch.cat([state[slot], x[r0:r0 + n].float()])          # [taps - 1 + n, W], oldest first
                k = self.spec.taps - 1
                out[r0:r0 + n] = sum(rows[k - i:k - i + n] @ self.w[i].t() for i in range(self.spec.taps))
                state[slot] = rows[-k:]
                r0 += n
            return out.to(x.dtype)

    @register_block("toy_post_norm")
    class PostNormBlock:
        cache_part = "attn"

        def __init__(self, spec, store, runtime):
            self.spec, self.rt = spec, runtime
            self.parts_ = {name: build_part(s, store, runtime) for name, s in spec.parts.items()}
            self.skip = float(spec.skip)

        def cache_spec(self):
            return self.parts_[self.spec.cache_part_name].cache_spec()

        def forward(self, stream, ctx, cache, owns_cache):
            x = stream.flush()
            p = self.parts_
            for part, norm in (("first", "norm_a"), ("ffn", "norm_b")):
                h = x.to(self.rt.dtype)
                y = p[part].forward(h, ctx, cache, owns_cache) if part == "first" else p[part].forward(h, ctx)
                y = y.float().sum(0) if y.dim() == 3 else y.float()
                out = torch.empty_like(h)
                p[norm].forward(x, out, delta=(self.skip * x + y).to(self.rt.dtype) - h, delta_scale=1.0)
                x.copy_(out.float())            # what the norm gave becomes the stream
            return stream

    class Arch:
        name = "Toy3ForCausalLM"
        model_types = ("toy3",)

        def read_config(self, obj):
            return dict(obj)

        def plan(self, c, present=None):
            def norm(n):
                return NormSpec("rms", W, 1e-5, {"weight": n})

            def ffn(p):
                return FeedForwardSpec("gated_mlp", W, {"gate": p + "g", "up": p + "u", "down": p + "d"}, inner=48)
            shift = MixerSpec("toy_shift", W, {"w0": "s.w0", "w1": "s.w1", "w2": "s.w2"}, taps=3)
            attn = MixerSpec("attention", W, {"q": "a.q", "k": "a.k", "v": "a.v", "o": "a.o"}, num_heads=2, num_kv_heads=2,
                             head_dim=HD, scale=HD ** -0.5, position=PositionSpec("rotary", HD, HD, 10000.0))
            layers = [BlockSpec("toy_post_norm", first=shift, norm_a=norm("l0.na"), ffn=ffn("l0."), norm_b=norm("l0.nb"),
                                skip=0.5, cache_part_name="first"),
                      BlockSpec("toy_post_norm", first=attn, norm_a=norm("l1.na"), ffn=ffn("l1."), norm_b=norm("l1.nb"),
                                skip=1.0, cache_part_name="first")]
            return ModelPlan(EmbeddingSpec(V, W, 1.0, {"weight": "emb"}), layers, [LayerRun(0), LayerRun(1)], norm("final"),
                             HeadSpec(V, W, True), 128)

    register_architecture(Arch())
    folder = str(tmp_path / "toy3")
    write_model_folder(folder, {"architectures": ["Toy3ForCausalLM"], "model_type": "toy3"}, 11, torch.float32)
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    toks = [int(t) for t in np.random.RandomState(5).randint(0, V, 45)]

    def reference():
        cfg = {"num_attention_heads": 2, "num_key_value_heads": 2, "head_dim": HD, "rope_theta": 10000.0,
               "partial_rotary_factor": 1.0, "attention_multiplier": 0.0}
        x = plain.embed(w["emb"], toks)
        n = len(toks)
        pad = np.concatenate([np.zeros((2, W)), x])
        y = sum(pad[2 - i:2 - i + n] @ w[f"s.w{i}"].T for i in range(3))
        x = plain.rms_norm(0.5 * x + y, w["l0.na"], 1e-5)
        x = plain.rms_norm(0.5 * x + plain.gated_mlp(x, w["l0.g"], w["l0.u"], w["l0.d"]), w["l0.nb"], 1e-5)
        aw = {"p.self_attn." + k + "_proj.weight": w["a." + k] for k in "qkvo"}
        x = plain.rms_norm(x + plain.attention_block(x, aw, "p.", cfg, np.arange(n)), w["l1.na"], 1e-5)
        x = plain.rms_norm(x + plain.gated_mlp(x, w["l1.g"], w["l1.u"], w["l1.d"]), w["l1.nb"], 1e-5)
        return plain.rms_norm(x, w["final"], 1e-5) @ w["emb"].T

    ref = reference()
    for cuts in ([45], [16, 7, 2, 1, 1, 18]):
        built = build(folder, dtype="float32", kv_tokens=128, max_batch_tokens=64, max_requests=2)
        assert set(built.cache.state_arrays) == {0} and len(built.cache.groups) == 1
        got, pos = [], 0
        for n in cuts:
            got.append(built.step_fn.step([StepEntry("r", toks[pos:pos + n], list(range(n)))]).cpu().numpy().copy())
            pos += n
        built.step_fn.end("r")
        err = np.abs(np.concatenate(got) - ref).max()
        assert err <= 3e-5 * max(1.0, np.abs(ref).max()), f"cuts {cuts}: {err}"


# ---------------------------------------------------------------------------------------------
# another position encoding and a feed-forward with routing, both defined here
# ---------------------------------------------------------------------------------------------

def _register_toy_parts():
    from dynalm_b200.parts import TensorDecl, register_feed_forward, register_position

    @register_position("toy_adjacent")
    class AdjacentPairs:
        """Rotates ADJACENT pairs (2i, 2i+1) by pos * theta^(-2i/d): no table for the fused kernel, so
        the attention mixer calls apply() before its cache write."""

        def __init__(self, spec, runtime):
            d = spec.head_dim
            self.inv = (spec.theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).to(runtime.device)

        def table(self):
            return None

        def apply(self, q, k, positions):
            ang = positions.double()[:, None] * self.inv[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for x in (q, k):
                if x is None:
                    continue
                a, b = x[..., 0::2].double(), x[..., 1::2].double()
                x[..., 0::2] = (a * c - b * s).to(x.dtype)
                x[..., 1::2] = (a * s + b * c).to(x.dtype)

    @register_feed_forward("toy_routed")
    class TopOneExperts:
        """Two experts, each a plain matrix; a token goes to the expert with the larger router logit
        (computed in float32) and is scaled by that logit's sigmoid."""

        @staticmethod
        def declare(spec):
            return {"router": TensorDecl((2, spec.width)), "e0": TensorDecl((spec.width, spec.width)),
                    "e1": TensorDecl((spec.width, spec.width))}

        def __init__(self, spec, tensors, runtime):
            self.t = tensors

        def forward(self, x, ctx):
            logits = x.float() @ self.t["router"].float().T
            pick = logits.argmax(-1)
            gate = torch.sigmoid(logits.gather(1, pick[:, None]))
            y0, y1 = x.float() @ self.t["e0"].float().T, x.float() @ self.t["e1"].float().T
            return (torch.where(pick[:, None] == 0, y0, y1) * gate).to(x.dtype)


def test_toy_position_encoding_and_routed_feed_forward(tmp_path):
    """A position encoding without a table (the mixer's apply() path) and a feed-forward with routing are
    registered from here, built into a model through a toy architecture, and stepped whole and cut."""
    _register_toy_parts()
    from dynalm_b200.config import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan,
                                    NormSpec, PositionSpec)
    from dynalm_b200.engine import StepEntry, build
    from dynalm_b200.registry import register_architecture
    from dynalm_b200.weights import write_model_folder

    W, V, HD = 64, 90, 32

    class Arch:
        name = "Toy2ForCausalLM"
        model_types = ("toy2",)

        def read_config(self, obj):
            return dict(obj)

        def plan(self, c, present=None):
            def norm(n):
                return NormSpec("rms", W, 1e-6, {"weight": n})
            layers = []
            for l in range(2):
                p = f"l{l}."
                layers.append(BlockSpec(
                    "pre_norm", mixer_norm=norm(p + "n1"),
                    mixer=MixerSpec("attention", W, {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o"}, num_heads=2,
                                    num_kv_heads=1, head_dim=HD, scale=HD ** -0.5,
                                    position=PositionSpec("toy_adjacent", HD, HD, 100.0)),
                    ffn_norm=norm(p + "n2"),
                    ffn=FeedForwardSpec("toy_routed", W, {"router": p + "r", "e0": p + "e0", "e1": p + "e1"})))
            return ModelPlan(EmbeddingSpec(V, W, 1.0, {"weight": "emb"}), layers, [LayerRun(0), LayerRun(1)], norm("final"),
                             HeadSpec(V, W, True), 128)

    register_architecture(Arch())
    folder = str(tmp_path / "toy2")
    write_model_folder(folder, {"architectures": ["Toy2ForCausalLM"], "model_type": "toy2"}, 6, torch.float32)
    w = plain.read_safetensors(os.path.join(folder, "model.safetensors"))
    toks = [int(t) for t in np.random.RandomState(3).randint(0, V, 45)]

    # plain reference
    n = len(toks)
    x = w["emb"][np.asarray(toks)]
    pos = np.arange(n)
    inv = 100.0 ** (-np.arange(0, HD, 2) / HD)
    ang = pos[:, None] * inv[None, :]

    def rot(t):
        a, b = t[..., 0::2], t[..., 1::2]
        out = np.empty_like(t)
        out[..., 0::2] = a * np.cos(ang)[:, None, :] - b * np.sin(ang)[:, None, :]
        out[..., 1::2] = a * np.sin(ang)[:, None, :] + b * np.cos(ang)[:, None, :]
        return out

    for l in range(2):
        p = f"l{l}."
        h = plain.rms_norm(x, w[p + "n1"], 1e-6)
        q = rot((h @ w[p + "q"].T).reshape(n, 2, HD))
        k = rot((h @ w[p + "k"].T).reshape(n, 1, HD))
        v = (h @ w[p + "v"].T).reshape(n, 1, HD)
        x = x + plain.attention(q, k, v, HD ** -0.5).reshape(n, 2 * HD) @ w[p + "o"].T
        h = plain.rms_norm(x, w[p + "n2"], 1e-6)
        logits = h @ w[p + "r"].T
        pick = logits.argmax(-1)
        gate = 1.0 / (1.0 + np.exp(-logits[np.arange(n), pick]))
        y = np.where(pick[:, None] == 0, h @ w[p + "e0"].T, h @ w[p + "e1"].T) * gate[:, None]
        x = x + y
    ref = plain.rms_norm(x, w["final"], 1e-6) @ w["emb"].T

    for cuts in ([45], [16, 7, 2, 5, 3, 2, 1, 1, 8]):
        built = build(folder, dtype="float32", kv_tokens=128, max_batch_tokens=64, max_requests=2)
        assert not built.model.graph_safe          # the toy feed-forward does not claim it, so nothing is captured
        got, p0 = [], 0
        for c in cuts:
            got.append(built.step_fn.step([StepEntry("r", toks[p0:p0 + c], list(range(c)))]).cpu().numpy().copy())
            p0 += c
        got = np.concatenate(got)
        assert np.abs(got - ref).max() <= 5e-5 * max(1.0, np.abs(ref).max()), f"cuts {cuts}"


def test_kernel_times_of_a_step(tiny_folders):
    """engine/profile.py: inside `kernel_times` a step runs launch by launch with every launch between two events;
    the table names the kernels with their counts, and the logits are those of the same step run as usual."""
    import numpy as np
    from tiny_configs import TINY
    from dynalm_b200.engine import StepEntry, build, profile
    cfg = TINY["b"][0]
    layers = cfg["num_hidden_layers"]
    rng = np.random.RandomState(3)
    prompt = [int(t) for t in rng.randint(0, cfg["vocab_size"], 40)]
    tail = [int(t) for t in rng.randint(0, cfg["vocab_size"], 5)]

    def run(profiled):
        built = build(tiny_folders["b"], dtype="bfloat16", kv_tokens=256, max_batch_tokens=64, max_requests=4)
        fn = built.step_fn
        fn.step([StepEntry("a", prompt, [])])
        if not profiled:
            return fn.step([StepEntry("a", tail[:1], [0]), StepEntry("b", tail, [4])]).float().cpu().numpy(), None
        with profile.kernel_times(fn) as times:
            logits = fn.step([StepEntry("a", tail[:1], [0]), StepEntry("b", tail, [4])]).float().cpu().numpy()
        return logits, times.totals()
    plain, _ = run(False)
    got, totals = run(True)
    assert np.array_equal(plain, got)
    assert totals["dl_rmsnorm"][0] == 2 * layers + 1 and totals["dl_embed"][0] == 1
    assert all(ms > 0.0 for _, ms in totals.values())
    assert "dl_rmsnorm" in profile.table(totals)


def test_kernel_times_measure_the_kernels():
    from dynalm_b200.kernels import ops
    """The events of `KernelTimes` stand on the stream the kernels run on: four launches of a product that takes a
    tenth of a millisecond are reported as about four times that, not as the few microseconds of their launches."""
    x = torch.randn(2048, 2048, device=DEV).to(torch.bfloat16)
    w = torch.randn(8192, 2048, device=DEV).to(torch.bfloat16)
    out = torch.empty(2048, 8192, dtype=torch.bfloat16, device=DEV)
    for _ in range(3):
        ops.gemm_tcgen05(x, w, out)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(4):
        ops.gemm_tcgen05(x, w, out)
    end.record()
    torch.cuda.synchronize()
    whole = begin.elapsed_time(end)
    with ops.KernelTimes() as times:
        for _ in range(4):
            ops.gemm_tcgen05(x, w, out)
    launches, ms = next(iter(times.totals().values()))
    assert launches == 4 and 0.5 * whole <= ms <= 3.0 * whole, (ms, whole)
