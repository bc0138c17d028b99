"""Command line in the manner of `dynalm run` (dynalm/src/cli/main.cpp:112-190, run.cpp:34-73,208-450).

    dynalm run <model_dir> --tokens 1,2,3 -n 32 --temp 0.8 --seed 4

Option names and meanings are the reference's where it has them (-n/--max-tokens, -c/--ctx, --batch,
--kv, --mode, --temp, --top-k, --top-p, --min-p, --repeat-penalty, --presence-penalty,
--frequency-penalty, --repeat-last-n, --seed, --no-stream, -q/-v). This engine starts at token ids:
the prompt is given as ids (`--tokens`, or `-p` holding ids separated by commas or spaces) or drawn
at random (`--prompt-len`); output is token ids. After the ids come the reference's two stats lines.
"""

from __future__ import annotations

import argparse
import contextlib
import os
import sys
import time

from .. import __version__
from ..utils import log

USAGE = """usage: dynalm [-q | -v | --log-level LEVEL] <command> [args]
       dynalm run <model> (--tokens IDS | -p IDS | --prompt-len N) [options]
       dynalm random-model <out_dir> --config FILE --seed S [--dtype bf16|f32]
       dynalm version
  <model>               a folder with config.json and model.safetensors
  --tokens IDS          prompt token ids, separated by commas (repeatable: one request each)
  -p, --prompt IDS      the same (this engine has no tokenizer; the prompt is ids)
  --prompt-len N        a random prompt of N ids drawn with --prompt-seed (default 0)
  -n, --max-tokens N    tokens to generate (default 128)
  -c, --ctx N           KV cache capacity in tokens (default 4096; auto = from the free device memory)
  --batch N             max tokens per forward pass (default 512)
  --kv bf16|f32         KV cache dtype; it follows the compute dtype (see --mode / --dtype)
  --mode M              auto | performance: bfloat16 kernels (default); exact | safe: everything in float32
  --dtype D             bf16 | f32: the same choice by name
  --max-running N       most requests decoded together (default 64)
  --chunk N             most prompt tokens of one request per step (default 128)
  --solo-prefill-chunk N  the same for a lone prompt in a step without decode rows (default 256; 0 = off)
  --stop-id ID          end-of-generation token id (repeatable)
  --no-stream           print only the final ids
sampling (default: greedy):
  --temp T              temperature (0 = greedy; also --temperature)
  --top-k K, --top-p P, --min-p P
  --repeat-penalty R, --presence-penalty P, --frequency-penalty F, --repeat-last-n N
  --seed S              RNG seed (reproducible output)
  --config FILE         options from a file (else $DYNALM_CONFIG, else ~/.dynalm/config.yaml): the reference's YAML
                        keys (runtime.context_length, runtime.batch_tokens, runtime.mode, kv_cache.dtype,
                        sampling.temperature, sampling.max_tokens, model.path) or lines `option = value`;
                        then DYNALM_CTX, DYNALM_BATCH, DYNALM_MODE, DYNALM_KV, DYNALM_TEMPERATURE,
                        DYNALM_MAX_TOKENS, DYNALM_MODEL; then the command line: later sources win
global: -q / --quiet (errors only), -v / --verbose, --log-level trace|debug|info|warn|error|off (default info, or
        $DYNALM_LOG_LEVEL), --version
"""


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def _run_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="dynalm run", add_help=False)
    ap.add_argument("model", nargs="?", default=None)
    ap.add_argument("--model", dest="model_option", default=None)
    ap.add_argument("--tokens", "-p", "--prompt", dest="tokens", action="append", default=[])
    ap.add_argument("--prompt-len", type=int, default=0)
    ap.add_argument("--prompt-seed", type=int, default=0)
    ap.add_argument("-n", "--max-tokens", type=int, default=128)
    ap.add_argument("-c", "--ctx", default="4096")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--kv", choices=["bf16", "f32", "f16"], default=None)
    ap.add_argument("--mode", choices=["auto", "performance", "exact", "safe"], default="auto")
    ap.add_argument("--dtype", choices=["bf16", "f32", "bfloat16", "float32"], default=None)
    ap.add_argument("--max-running", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--solo-prefill-chunk", type=int, default=256)
    ap.add_argument("--stop-id", type=int, action="append", default=[])
    ap.add_argument("--no-stream", action="store_true")
    ap.add_argument("--temp", "--temperature", dest="temp", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--repeat-last-n", type=int, default=64)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("-h", "--help", action="store_true")
    return ap


# what `run` takes from the config file and from DYNALM_* (the reference's kRunConfigOptions,
# dynalm/src/cli/run.cpp:202-207, as far as this engine has the option): name -> takes a value
RUN_CONFIG_OPTIONS = {"model": True, "ctx": True, "batch": True, "kv": True, "mode": True, "temperature": True,
                      "max-tokens": True}


def cmd_run(argv, env=None) -> int:
    from ..errors import EngineError
    from .config import merge_config
    try:
        argv = merge_config(argv, RUN_CONFIG_OPTIONS, env)
    except EngineError as e:
        print(f"run: {e}", file=sys.stderr)
        return 1
    args = _run_parser().parse_args(argv)
    if args.help:
        sys.stderr.write(USAGE)
        return 0
    args.model = args.model or args.model_option
    if args.model is None:
        sys.stderr.write(USAGE)
        return 2
    if args.ctx == "auto":
        args.ctx = None              # sized from the free device memory
    else:
        try:
            args.ctx = int(args.ctx)
            if args.ctx <= 0:
                raise ValueError
        except ValueError:
            print(f"dynalm: --ctx takes a positive number of tokens or 'auto', not '{args.ctx}'", file=sys.stderr)
            return 2
    import numpy as np
    from ..engine import Engine, SchedulerConfig
    from ..sampling import SamplingParams

    dtype = "float32" if (args.dtype in ("f32", "float32") or args.mode in ("exact", "safe")) else "bfloat16"
    if args.kv == "f32" and dtype != "float32":
        print("dynalm: --kv f32 needs --mode exact (the cache has the compute dtype)", file=sys.stderr)
        return 2
    if args.kv == "f16":
        print("dynalm: --kv f16 is not offered; the cache is bf16 (or f32 with --mode exact)", file=sys.stderr)
        return 2
    try:
        sched = SchedulerConfig(max_running=args.max_running, max_prefill_chunk=args.chunk, max_batch_tokens=args.batch,
                                solo_prefill_chunk=args.solo_prefill_chunk)
        engine = Engine(args.model, dtype=dtype, ctx=args.ctx, batch=args.batch, max_running=args.max_running,
                        scheduler=sched)
    except EngineError as e:
        print(f"dynalm: {e}", file=sys.stderr)
        return 1
    prompts = [_ids(t) for t in args.tokens]
    if args.prompt_len > 0:
        rng = np.random.RandomState(args.prompt_seed)
        prompts.append([int(t) for t in rng.randint(0, engine.config.vocab_size, size=args.prompt_len)])
    if not prompts:
        sys.stderr.write(USAGE)
        return 2
    sp = [SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                         repetition_penalty=args.repeat_penalty, presence_penalty=args.presence_penalty,
                         frequency_penalty=args.frequency_penalty, penalty_last_n=args.repeat_last_n,
                         seed=None if args.seed is None else args.seed + i) for i in range(len(prompts))]
    from ..engine import profile
    timing = (profile.kernel_times(engine.executor.step_fn) if os.environ.get("DYNALM_FORWARD_PROFILE", "0") != "0"
              else contextlib.nullcontext())
    with timing as kernel_times:
        rc = _generate(args, engine, prompts, sp)
    if kernel_times is not None:
        log.info("kernels", "\n" + profile.table(kernel_times.totals()))
    return rc


def _generate(args, engine, prompts, sp) -> int:
    from ..engine import Request
    t0 = time.perf_counter()
    ids = [engine.scheduler.submit(Request(p, args.max_tokens, s, tuple(args.stop_id))) for p, s in zip(prompts, sp)]
    out = {i: [] for i in ids}
    final = {}
    ttft = None
    gaps = []
    last = t0
    while not engine.scheduler.idle:
        for ev in engine.scheduler.step():
            now = time.perf_counter()
            if ev.token is not None:
                out[ev.request_id].append(ev.token)
                if ttft is None:
                    ttft = (now - t0) * 1e3
                else:
                    gaps.append((now - last) * 1e3)
                last = now
                if not args.no_stream and len(ids) == 1:
                    sys.stdout.write(f"{ev.token} ")
                    sys.stdout.flush()
            if ev.finished:
                final[ev.request_id] = ev
    total_ms = (time.perf_counter() - t0) * 1e3
    if not args.no_stream and len(ids) == 1:
        sys.stdout.write("\n")
    else:
        for i in ids:
            print(" ".join(str(t) for t in out[i]))
    rc = 0
    for i in ids:
        if final[i].error:
            print(f"dynalm: request {i}: {final[i].error}", file=sys.stderr)
            rc = 1
    if log.enabled(log.INFO):
        gaps.sort()

        def pct(p):
            return gaps[min(len(gaps) - 1, int(p / 100.0 * len(gaps)))] if gaps else 0.0
        n_prompt = sum(len(p) for p in prompts)
        n_gen = sum(len(v) for v in out.values())
        decode_s = (total_ms - (ttft or 0.0)) / 1e3
        reason = ",".join(sorted({str(final[i].finish_reason or final[i].status) for i in ids}))
        log.info("stats", f"prompt {n_prompt} tok | TTFT {ttft or 0.0:.1f} ms | generated {n_gen} tok, "
                 f"{(n_gen - len(ids)) / decode_s if decode_s > 0 else 0.0:.1f} tok/s | finish {reason} | "
                 f"inter-delta p50 {pct(50):.1f} p90 {pct(90):.1f} p99 {pct(99):.1f} ms")
        ss = engine.scheduler.stats
        if ss.steps_decode_only > 0:
            log.info("engine", f"prefill {ss.forward_prefill_only_ms + ss.forward_mixed_ms:.1f} ms (forward, "
                     f"{ss.steps_prefill_only + ss.steps_mixed} steps) | decode step "
                     f"{ss.forward_decode_only_ms / ss.steps_decode_only:.2f} ms (forward, {ss.steps_decode_only} steps)")
        st = engine.stats()
        log.debug("engine", f"cache {st['pages']} pages ({st['cache_bytes'] / 2**20:.0f} MiB), workspace "
                  f"{st['workspace_bytes'] / 2**20:.0f} MiB, {st['kernel_launches']} kernel launches, "
                  f"{st['library_products']} library products, {st['graphs']['captured']} graphs captured")
    return rc


def cmd_random_model(argv) -> int:
    ap = argparse.ArgumentParser(prog="dynalm random-model")
    ap.add_argument("out_dir")
    ap.add_argument("--config", required=True, help="a config.json to copy sizes from")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", choices=["bf16", "f32"], default="bf16")
    args = ap.parse_args(argv)
    import torch
    from ..config.reader import read_json_file
    from ..weights import write_model_folder
    write_model_folder(args.out_dir, read_json_file(args.config), args.seed,
                       torch.bfloat16 if args.dtype == "bf16" else torch.float32)
    print(args.out_dir)
    return 0


def main(argv=None) -> int:
    """Global options come before the command (dynalm/src/cli/main.cpp:118-151): -q / --quiet (errors only),
    -v / --verbose (debug), --log-level trace|debug|info|warn|error|off|quiet|normal|verbose; DYNALM_LOG_LEVEL sets
    the default."""
    argv = list(sys.argv[1:] if argv is None else argv)
    while argv and argv[0].startswith("-") and argv[0] not in ("-h", "--help"):
        flag = argv.pop(0)
        if flag == "--version":
            print(f"dynalm_b200 {__version__}")
            return 0
        if flag == "--log-level" and argv:
            name = argv.pop(0)
            if not log.set_level(name):
                print(f"dynalm: invalid log level '{name}' (quiet, normal, verbose, debug, trace)", file=sys.stderr)
                return 1
        elif flag.startswith("--log-level="):
            if not log.set_level(flag.split("=", 1)[1]):
                print(f"dynalm: invalid log level '{flag.split('=', 1)[1]}' (quiet, normal, verbose, debug, trace)",
                      file=sys.stderr)
                return 1
        elif flag in ("-q", "--quiet"):
            log.set_level("quiet")
        elif flag in ("-v", "--verbose"):
            log.set_level("verbose")
        else:
            print(f"dynalm: unknown option '{flag}'", file=sys.stderr)
            return 1
    if not argv or argv[0] in ("-h", "--help", "help"):
        sys.stderr.write(USAGE)
        return 0 if argv else 2
    cmd, rest = argv[0], argv[1:]
    if cmd == "run":
        return cmd_run(rest)
    if cmd == "random-model":
        return cmd_random_model(rest)
    if cmd == "version":
        print(f"dynalm_b200 {__version__}")
        return 0
    print(f"dynalm: unknown command '{cmd}'\n", file=sys.stderr)
    sys.stderr.write(USAGE)
    return 2


if __name__ == "__main__":
    sys.exit(main())
