"""Decode and prefill throughput of dynalm_b200 on one B200, Llama 3.2 1B shape, random bf16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 requests that each hold 2,048 tokens of context. `value` is
decoded tokens per second over exactly K steps, timed with CUDA events on the launching stream (the
token ids fed are fixed, nothing is read back inside the timed region), the median of --repeats (5) such
measurements with the slowest and the fastest in `spread`; `e2e` is the same through the Python entry
point's scheduler: host token ids in, sampled token ids out, every step. Beside them: a 2,048-token
prefill with its fraction of the bf16 matrix peak, the decode step's fraction of the HBM roofline (every
weight read once plus the cache of the live requests), and as `points` decode at batch 1 and 64, decode
at batch 1, 8 and 64 with about 8,000 tokens of context each (as many as the 8,192-token benchmark context
leaves room for while the measurement grows them), and a prefill of 8,192 tokens, each with its fraction
of the roofline; last, the continuous-batching workloads of the 3B and 8B shapes (tokens/s over the whole run,
median time to the first token, decode-only step), a 32,768-token prompt brought in portions of 512, and the
end-to-end decode again with requests that draw their tokens (temperature, top-k, top-p, a penalty). `--workload serve3b | serve8b` runs one of those alone and
prints its full record. Prints one JSON line.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama 3.2 1B shape.
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "tie_word_embeddings": True,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
}
# BASELINE.json configs[3] and [4]: the 3B and 8B shapes with their serving workloads.
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, num_key_value_heads=8,
                head_dim=128, intermediate_size=8192)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SERVING = {
    # name: (config, weight seed, requests, prompt lengths (lo, hi), prompt seed, decode tokens, prefill chunk)
    "serve3b": (LLAMA_3B, 5, 32, (128, 4096), 6, 256, 512),
    "serve8b": (LLAMA_8B, 7, 64, (1024, 1024), 8, 512, 512),
}
FULL_LAYERS = 16
CONTEXT = 8192          # benchmark context length: the longest a request may grow
HELD = 2048             # tokens each sequence holds when decoding
PREFILL_TOKENS = 2048
LONG_PREFILL = 8192     # a further point: one prompt of the whole benchmark context
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in the background during the timed region: SM clocks and throttle reasons."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if mhz:
            self.result = {"sm_mhz": statistics.median(mhz), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def weight_bytes(cfg, layers):
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qw = cfg["num_attention_heads"] * cfg["head_dim"]
    kw = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (qw + 2 * kw) * H + H * qw + 3 * F * H
    return 2 * (layers * per_layer + V * H) + 4 * H * (2 * layers + 1)      # bf16 matrices, fp32 norm weights


def kv_bytes_per_token(cfg, layers):
    return 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * layers * 2


def prefill_flops(cfg, layers, T):
    H, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, hd = cfg["num_attention_heads"], cfg["head_dim"]
    qw, kw = nh * hd, cfg["num_key_value_heads"] * hd
    per_layer = (qw + 2 * kw) * H + H * qw + 3 * F * H
    return 2.0 * layers * per_layer * T + 4.0 * nh * hd * layers * T * (T + 1) / 2 + 2.0 * V * H


def write_random_llama(folder, cfg, seed):
    """config.json and model.safetensors (bfloat16, N(0, 0.02) matrices, norm weights 1 + N(0, 0.1)) for the reference
    arm, written with NumPy alone: that arm imports nothing of dynalm_b200."""
    import numpy as np
    H, F, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    qw, kw = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    shapes = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", True):
        shapes["lm_head.weight"] = (V, H)
    for l in range(L):
        p = f"model.layers.{l}."
        shapes.update({p + "input_layernorm.weight": (H,), p + "post_attention_layernorm.weight": (H,),
                       p + "self_attn.q_proj.weight": (qw, H), p + "self_attn.k_proj.weight": (kw, H),
                       p + "self_attn.v_proj.weight": (kw, H), p + "self_attn.o_proj.weight": (H, qw),
                       p + "mlp.gate_proj.weight": (F, H), p + "mlp.up_proj.weight": (F, H),
                       p + "mlp.down_proj.weight": (H, F)})
    header, off = {}, 0
    for name, shape in shapes.items():
        n = 2 * int(np.prod(shape))
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    from concurrent.futures import ThreadPoolExecutor
    PIECE = 1 << 22

    def piece(job):
        index, m, vector = job
        x = np.random.default_rng([seed, index]).standard_normal(m, dtype=np.float32)
        x = x * np.float32(0.1) + np.float32(1.0) if vector else x * np.float32(0.02)
        bits = x.view(np.uint32)
        bits = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)    # round to nearest even
        return bits.astype("<u2").tobytes()

    jobs = []
    for name, shape in shapes.items():
        n = int(np.prod(shape))
        jobs += [(len(jobs) + k, min(PIECE, n - i), len(shape) == 1) for k, i in enumerate(range(0, n, PIECE))]
    with open(os.path.join(folder, "model.safetensors"), "wb") as f, ThreadPoolExecutor(os.cpu_count() or 4) as pool:
        f.write(len(text).to_bytes(8, "little"))
        f.write(text)
        for data in pool.map(piece, jobs):
            f.write(data)


def reference_arm(args):
    """`--impl reference`: the same metric from dynalm-project/dynalm's own engine, unmodified, through its public C++
    API on its CPU device (it has no CUDA code of its own; its GPU backends are ggml's and are fetched from the
    network when the project is configured). baseline/build_reference.sh builds the program on a machine that has
    the reference's source; here it is only run. Nothing of dynalm_b200 is imported on this path."""
    import tempfile
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_bench")

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    if args.gpus != 1:
        return unavailable("the reference arm is the reference's CPU engine: one process, no GPUs")
    if not os.path.isfile(exe):
        return unavailable("baseline/_ref/ref_bench is not built (sh baseline/build_reference.sh <reference source>); "
                           "pip cannot install the reference: it is a C++/CMake project without setup.py or pyproject.toml")
    W, K = max(3, args.warmup), max(1, args.steps)
    cfg = dict(LLAMA_1B)
    cfg["num_hidden_layers"] = args.layers
    points = "-" if args.no_points else ",".join(str(b) for b in sorted({1, 64} - {args.batch}))
    point_steps = min(K, 8)       # batch 64 takes about a second a step on a CPU
    with tempfile.TemporaryDirectory(prefix="dynalm_ref_") as d:
        t0 = time.time()
        write_random_llama(d, cfg, 0)
        print(f"[bench] reference arm: model folder written in {time.time() - t0:.1f} s", file=sys.stderr)
        try:
            proc = subprocess.run([exe, d, str(args.batch), str(HELD), str(K), str(W), str(PREFILL_TOKENS), points, str(point_steps), "0"],
                                  capture_output=True, text=True, timeout=3000)
        except (OSError, subprocess.TimeoutExpired) as e:
            return unavailable(f"baseline/_ref/ref_bench could not be run: {e}")
    if proc.returncode != 0:
        return unavailable(f"baseline/_ref/ref_bench exited with {proc.returncode}: {proc.stderr.strip()[-300:]}")
    r = json.loads(proc.stdout.strip().splitlines()[-1])
    ms = r["decode_ms_per_step"]
    out = {
        "metric": "decode tokens/s, Llama 3.2 1B shape, batch 8, 2048 tokens of context per sequence",
        "value": round(args.batch / ms * 1e3, 2), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights, fp32 activations, f16 cache (the reference's defaults)",
        "data": "synthetic: random weights N(0, 0.02) seed 0, random token ids",
        "config": {"model": "llama-3.2-1b-shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": 2048,
                   "heads": 32, "kv_heads": 8, "head_dim": 64, "intermediate": 8192, "vocab": 128256,
                   "global_batch": args.batch, "seq_len": HELD, "context": CONTEXT, "kv_block": 16, "parallelism": "none",
                   "device": f"the reference's CPU device ({r['device']}, {r['threads']} threads): it has no CUDA code",
                   "tied_embeddings": True},
        "e2e": {"value": round(r["e2e_tokens_per_s"], 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0, "through": "the reference's Scheduler: token ids in, token callbacks out"},
        "gpu_launches": 0,
        "prefill": {"value": round(PREFILL_TOKENS / r["prefill_ms"] * 1e3, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(r["prefill_ms"], 1)},
        "points": {f"decode_b{b}": round(int(b) / v * 1e3, 2) for b, v in r["points_ms_per_step"].items()
                   if int(b) != args.batch},
        "impl": "reference",
    }
    print(json.dumps(out))
    return 0


def serving(name, layers=None, emit=True):
    """Continuous batching end to end through the Python entry point: all requests submitted at once, prompts
    prefilled in chunks beside decode rows, every request decoding its full count. Prints one JSON line, or
    (emit=False) returns the record."""
    import numpy as np
    import torch
    from dynalm_b200 import Engine, Request, SchedulerConfig

    cfg, wseed, n_req, (lo, hi), pseed, n_decode, chunk = SERVING[name]
    cfg = dict(cfg)
    full_layers = cfg["num_hidden_layers"]
    if layers:
        cfg["num_hidden_layers"] = layers
    rng = np.random.RandomState(pseed)
    lens = [int(rng.randint(lo, hi + 1)) for _ in range(n_req)]
    prompts = [[int(t) for t in rng.randint(0, cfg["vocab_size"], n)] for n in lens]
    kv_tokens = sum(-(-(n + n_decode) // 16) * 16 for n in lens) + 1024
    t0 = time.time()
    eng = Engine(config=cfg, random_seed=wseed, dtype="bfloat16", ctx=kv_tokens, batch=chunk + n_req, max_running=n_req,
                 scheduler=SchedulerConfig(max_running=n_req, decode_token_budget=n_req, prefill_token_budget=chunk,
                                           max_prefill_chunk=chunk, max_batch_tokens=chunk + n_req))
    print(f"[bench] {name}: engine built in {time.time() - t0:.1f} s", file=sys.stderr)
    warm = eng.generate(prompts[0][:64], max_tokens=4)          # loads kernels, captures nothing of the timed run
    assert len(warm.tokens) == 4
    for p in prompts:
        eng.scheduler.submit(Request(p, max_new_tokens=n_decode))
    done, first, n_tok = 0, {}, 0
    torch.cuda.synchronize()
    with ClockSampler() as cs:
        t0 = time.perf_counter()
        while not eng.scheduler.idle:
            for ev in eng.scheduler.step():
                if ev.token is not None:
                    n_tok += 1
                    first.setdefault(ev.request_id, time.perf_counter() - t0)
                done += ev.finished
        torch.cuda.synchronize()
        total = time.perf_counter() - t0
    st = eng.scheduler.stats
    ttft = sorted(first.values())
    out = {
        "metric": f"continuous batching, {name}: generated tokens/s over the whole run", "value": round(n_tok / total, 1),
        "unit": "tokens/s", "n_gpus": 1, "impl": "ours", "dtype": "bf16", "seconds": round(total, 3),
        "requests": n_req, "finished": done, "generated": n_tok, "prompt_tokens": sum(lens),
        "prompt_tokens_per_s": round(sum(lens) / total, 1),
        "ttft_ms": {"p50": round(ttft[len(ttft) // 2] * 1e3, 1), "max": round(ttft[-1] * 1e3, 1)},
        "steps": {"decode_only": st.steps_decode_only, "prefill_only": st.steps_prefill_only, "mixed": st.steps_mixed},
        "decode_step_ms": round(st.forward_decode_only_ms / max(1, st.steps_decode_only), 3),
        "preemptions": st.preemptions,
        "config": {"model": name, "layers": cfg["num_hidden_layers"], "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "prefill_chunk": chunk,
                   "decode_tokens": n_decode, "kv_tokens": kv_tokens},
        "clocks": cs.result, "data": "synthetic: random weights, random token ids",
    }
    if not emit:
        del eng
        return out
    print(json.dumps(out))
    return 0


def long_prompt(tokens=32768, portion=512):
    """One prompt of `tokens` tokens brought in portions of `portion` through the step function (the 1B shape with the
    131,072 positions the model has): tokens/s. What a long request costs a server that cuts prompts into portions:
    every portion's attention walks all keys so far."""
    import numpy as np
    import torch
    from dynalm_b200 import Engine, StepEntry
    cfg = dict(LLAMA_1B)
    cfg["max_position_embeddings"] = 131072
    eng = Engine(config=cfg, random_seed=0, dtype="bfloat16", ctx=tokens + 1024, batch=max(portion, 512), max_running=2)
    rng = np.random.RandomState(1)
    ids = [int(t) for t in rng.randint(0, cfg["vocab_size"], tokens)]

    def once(name):
        for p in range(0, tokens, portion):
            eng.step_fn.step([StepEntry(name, ids[p:p + portion], [len(ids[p:p + portion]) - 1] if p + portion >= tokens else [])])
        eng.step_fn.end(name)
    once("warm")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    once("timed")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    del eng
    return round(tokens / dt, 1), round(dt * 1e3, 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--workload", choices=["decode"] + sorted(SERVING), default="decode",
                    help="decode: the default benchmark; serve3b / serve8b: continuous batching of the 3B / 8B workloads")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-long", action="store_true", help="skip the points at 8,192 tokens (prefill and decode)")
    ap.add_argument("--no-serve", action="store_true", help="skip the points of the 3B and 8B serving workloads")
    ap.add_argument("--repeats", type=int, default=5, help="the timed K steps are repeated this often; `value` is the median")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profiling)")
    ap.add_argument("--only", choices=["all", "decode", "prefill"], default="all",
                    help="profiling aid: run only the device-timed decode loop, or only the prefill")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.workload != "decode":
        return serving(args.workload, args.layers if args.layers != FULL_LAYERS else None)
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import numpy as np
    import torch
    from dynalm_b200 import Engine, Request, SchedulerConfig, StepEntry
    from dynalm_b200.kernels import gemm, ops

    peaks = load_peaks()
    cfg = dict(LLAMA_1B)
    cfg["num_hidden_layers"] = args.layers
    R = max(1, args.repeats)
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    long_batches = [] if (args.no_points or args.no_long) else sorted({1, args.batch, 64})
    max_b = max(batches)
    PRIME_MAX = 8
    span = PRIME_MAX + W + R * K + 4 * args.batch + 96          # tokens a sequence grows by while it is measured
    held_long = CONTEXT - span - 16                             # "8,192 tokens of context": as many as fit under it
    kv_tokens = max(max_b * (-(-(HELD + span) // 16) * 16),
                    max(long_batches, default=0) * (-(-CONTEXT // 16) * 16)) + 2 * LONG_PREFILL + 4096
    t_build = time.time()
    eng = Engine(config=cfg, random_seed=0, dtype="bfloat16", ctx=kv_tokens,
                 batch=LONG_PREFILL if not args.no_long else PREFILL_TOKENS, max_running=max_b,
                 scheduler=SchedulerConfig(max_running=max_b, decode_token_budget=max_b,
                                           prefill_token_budget=PREFILL_TOKENS - max_b,
                                           max_prefill_chunk=PREFILL_TOKENS - max_b, max_batch_tokens=PREFILL_TOKENS))
    step_fn = eng.step_fn
    if args.no_graphs:
        step_fn.use_graphs = False
    rng = np.random.RandomState(0)
    vocab = cfg["vocab_size"]
    print(f"[bench] engine built in {time.time() - t_build:.1f} s ({args.layers} layers)", file=sys.stderr)

    def timed(fn, n, lead=None):
        """n calls of fn between two CUDA events on the current stream -> milliseconds (`lead`: issued, untimed, just
        before the first event)."""
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if lead is not None:
            lead()
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    # ---- prefill of one prompt of 2,048 tokens (and of 8,192) ---------------------------------------------------
    def prefill_point(T, reps):
        prompt = [int(t) for t in rng.randint(0, vocab, T)]

        def once():
            step_fn.step([StepEntry("p", prompt, [T - 1])])
            step_fn.end("p")
        for _ in range(3):
            once()
        # an untimed prompt goes in front of each measurement: the timed region then begins with the GPU busy and the
        # host already queuing the next prompt, instead of with the GPU waiting for the host's first launch
        ms = statistics.median(timed(once, 3, lead=once) / 3 for _ in range(reps))
        flops = prefill_flops(cfg, args.layers, T)
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    prefill = prefill_point(PREFILL_TOKENS, R) if args.only != "decode" else None
    if args.only == "prefill":
        print(json.dumps({"prefill": prefill, "prefill_long": None if args.no_long else prefill_point(LONG_PREFILL, 3)}))
        return 0
    prefill_long = prefill_point(LONG_PREFILL, 3) if (args.only == "all" and not args.no_long and not args.no_points) else None

    # ---- decode: device-timed ------------------------------------------------------------------------------
    def fill(B, held):
        for r in range(B):
            left = held
            while left > 0:            # a long context comes in portions the engine's step takes
                n = min(left, step_fn.max_tokens)
                step_fn.step([StepEntry(("d", r), [int(t) for t in rng.randint(0, vocab, n)], [])])
                left -= n

    def drop(B):
        for r in range(B):
            step_fn.end(("d", r))

    ids_out = torch.zeros(max_b, dtype=torch.int32, device="cuda:0")
    # the step function captures a decode-only launch shape as a CUDA graph when it has come GRAPH_AFTER times: that
    # many steps of setup come before the warm-up, so that warm-up and timed steps are the steady state
    PRIME = min(PRIME_MAX, step_fn.GRAPH_AFTER) if step_fn.use_graphs else 0
    launches = lib_calls = 0
    clocks = None

    def decode_point(B, held, main=False):
        """R repeats of K timed decode steps of B sequences that hold `held` tokens -> (ms per step of each repeat,
        tokens every sequence held in the middle of the measurement)."""
        nonlocal launches, lib_calls, clocks
        fill(B, held)
        toks = [[int(rng.randint(0, vocab))] for _ in range(B)]

        def decode_once():
            # greedy: the head picks the most likely token in its product's epilogue where it can
            logits = step_fn.step([StepEntry(("d", r), toks[r], [0]) for r in range(B)], choose=(ids_out[:B], None))
            if logits is not None:
                ops.argmax(logits, ids_out[:B])
        for _ in range(PRIME + W):       # PRIME steps of setup (the launch shape becomes a CUDA graph), then W of warm-up
            decode_once()
        reps = []
        if main:
            l0, g0, r0 = ops.LAUNCHES, gemm.LIBRARY_CALLS, getattr(step_fn, "graph_kernel_launches", 0)
            with ClockSampler() as cs:
                for _ in range(R):
                    reps.append(timed(decode_once, K) / K)
            clocks = cs.result
            launches = (ops.LAUNCHES - l0 + getattr(step_fn, "graph_kernel_launches", 0) - r0) // R
            lib_calls = (gemm.LIBRARY_CALLS - g0) // R
        else:
            steps = K if B <= 16 else min(K, 32)
            for _ in range(min(R, 3)):
                reps.append(timed(decode_once, steps) / steps)
            mid = held + PRIME + W + len(reps) * steps / 2
            drop(B)
            return reps, mid
        drop(B)
        return reps, held + PRIME + W + R * K / 2

    def frac_of_roofline(B, ms, mid):
        bytes_step = weight_bytes(cfg, args.layers) + B * mid * kv_bytes_per_token(cfg, args.layers)
        return bytes_step / (ms * 1e-3) / 1e9

    points = {}
    main_reps, main_mid = decode_point(args.batch, HELD, main=True)
    for B in batches:
        if B != args.batch:
            reps, mid = decode_point(B, HELD)
            ms = statistics.median(reps)
            points[f"decode_b{B}"] = round(B / ms * 1e3, 1)
            points[f"decode_b{B}_frac"] = round(frac_of_roofline(B, ms, mid) / peaks["hbm_gbs"], 4)
    for B in long_batches:
        reps, mid = decode_point(B, held_long)
        ms = statistics.median(reps)
        points[f"decode_b{B}_ctx8k"] = round(B / ms * 1e3, 1)
        points[f"decode_b{B}_ctx8k_frac"] = round(frac_of_roofline(B, ms, mid) / peaks["hbm_gbs"], 4)
    if prefill_long is not None:
        points["prefill_8192"] = prefill_long["value"]
        points["prefill_8192_frac"] = prefill_long["frac"]

    ms_step = statistics.median(main_reps)
    value = args.batch / ms_step * 1e3
    achieved = frac_of_roofline(args.batch, ms_step, main_mid)
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}
    spread = {"repeats": len(main_reps), "min": round(args.batch / max(main_reps) * 1e3, 1),
              "max": round(args.batch / min(main_reps) * 1e3, 1)}

    if args.only == "decode":
        print(json.dumps({"decode_ms_per_step": ms_step, "spread": spread, "roofline": roofline, "points": points}))
        return 0

    # ---- decode end to end through the scheduler: host ids in, host ids out, every step ----------------------
    B = args.batch
    for r in range(B):
        eng.scheduler.submit(Request([int(t) for t in rng.randint(0, vocab, HELD)], max_new_tokens=span - 8))
    while not eng.scheduler.idle and (any(s.status != "decode" or s.pending != 1 for s in eng.scheduler.running)
                                      or eng.scheduler.waiting or eng.scheduler.incoming or not eng.scheduler.running):
        eng.scheduler.step()
    for _ in range(PRIME + W):
        eng.scheduler.step()
    h0, d0 = eng.executor.h2d_bytes, eng.executor.d2h_bytes
    e2e_reps = []
    for _ in range(R):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_tok = 0
        for _ in range(K):
            n_tok += sum(1 for ev in eng.scheduler.step() if ev.token is not None)
        torch.cuda.synchronize()
        e2e_reps.append(n_tok / (time.perf_counter() - t0))
    e2e = {"value": round(statistics.median(e2e_reps), 1), "unit": "tokens/s",
           "h2d_bytes_per_step": (eng.executor.h2d_bytes - h0) // (R * K),
           "d2h_bytes_per_step": (eng.executor.d2h_bytes - d0) // (R * K),
           "min": round(min(e2e_reps), 1), "max": round(max(e2e_reps), 1)}
    for s_ in list(eng.scheduler.running):
        eng.scheduler.cancel(s_.id)
    while not eng.scheduler.idle:
        eng.scheduler.step()

    # ---- the same end to end with requests that draw their tokens: through the sampling kernels, ids out ---------
    if not args.no_points:
        from dynalm_b200 import SamplingParams
        drawn = {"temperature": dict(temperature=0.8), "top_k40": dict(temperature=0.8, top_k=40),
                 "top_p0.9": dict(temperature=0.8, top_p=0.9),
                 "top_k40_top_p0.9_penalty": dict(temperature=0.8, top_k=40, top_p=0.9, repetition_penalty=1.1)}
        for name, how in drawn.items():
            try:
                for r in range(B):
                    eng.scheduler.submit(Request([int(t) for t in rng.randint(0, vocab, HELD)], max_new_tokens=span - 8,
                                                 sampling=SamplingParams(seed=r, **how)))
                while not eng.scheduler.idle and (any(s.status != "decode" or s.pending != 1 for s in eng.scheduler.running)
                                                  or eng.scheduler.waiting or eng.scheduler.incoming
                                                  or not eng.scheduler.running):
                    eng.scheduler.step()
                for _ in range(PRIME + W):
                    eng.scheduler.step()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                n_tok = 0
                for _ in range(K):
                    n_tok += sum(1 for ev in eng.scheduler.step() if ev.token is not None)
                torch.cuda.synchronize()
                points[f"e2e_b{B}_{name}"] = round(n_tok / (time.perf_counter() - t0), 1)
            except Exception as e:           # a point that fails does not take the line with it
                points[f"e2e_b{B}_{name}_error"] = f"{type(e).__name__}: {e}"[:200]
            for s_ in list(eng.scheduler.running):
                eng.scheduler.cancel(s_.id)
            while not eng.scheduler.idle:
                eng.scheduler.step()
        points["rows_sampled_on_the_host"] = eng.executor.host_sampled

    # ---- the serving workloads of the larger shapes, as points (each builds its own engine) ---------------------
    if not (args.no_points or args.no_serve or args.layers != FULL_LAYERS):
        import gc
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        for name in sorted(SERVING):
            try:
                got = serving(name, emit=False)
                points[f"{name}_tokens_per_s"] = got["value"]
                points[f"{name}_ttft_p50_ms"] = got["ttft_ms"]["p50"]
                points[f"{name}_decode_step_ms"] = got["decode_step_ms"]
            except Exception as e:           # a point that fails does not take the line with it
                points[f"{name}_error"] = f"{type(e).__name__}: {e}"[:200]
            gc.collect()
            torch.cuda.empty_cache()
        try:
            points["prefill_32768_in_portions_of_512"], points["prefill_32768_in_portions_of_512_ms"] = long_prompt()
        except Exception as e:
            points["prefill_32768_in_portions_of_512_error"] = f"{type(e).__name__}: {e}"[:200]
        gc.collect()
        torch.cuda.empty_cache()

    out = {
        "metric": "decode tokens/s, Llama 3.2 1B shape, batch 8, 2048 tokens of context per sequence",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, random token ids",
        "config": {"model": "llama-3.2-1b-shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": 2048,
                   "heads": 32, "kv_heads": 8, "head_dim": 64, "intermediate": 8192, "vocab": 128256,
                   "global_batch": args.batch, "seq_len": HELD, "context": CONTEXT, "kv_block": 16, "parallelism": "none",
                   "l2": "inputs larger than L2 (weights + cache >= 2.5 GB per step)", "tied_embeddings": True,
                   "value_is": f"median of {len(main_reps)} repeats of {K} steps", "ctx8k_points_hold": held_long},
        "spread": spread, "e2e": e2e, "gpu_launches": launches, "library_gemm_calls": lib_calls, "prefill": prefill,
        "roofline": roofline, "points": points, "clocks": clocks, "impl": "ours",
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
