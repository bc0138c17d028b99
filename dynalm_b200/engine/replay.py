"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns nothing: the model, the step function, the cache and the kernels are
the ones generation uses. The reference's counterparts are its accuracy bench, which steps the
model one token at a time, in chunks and two sequences per batch
(dynalm/benchmarks/bench_gpu_accuracy.cpp:232-237,280-302,346-388), and tools/ref_model.py.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: for each request its next tokens and the places among them whose logits are wanted; all
entries of a step run as one batch. `end`: requests that are finished after this step. For a step
that wants something, `<out>/<step>.f32` receives the logits [wanted, vocab] as little-endian
float32, in the order of the entries and of `want`. After every step a line `done <step>` is printed.

`--summary FILE` adds a text line per wanted place, with what tools/ref_model.py of the reference reports of a
logits row (:236-247): the id of the largest logit (ties: the lowest id), the 8 largest as id:logit, and the sum and
the sum of squares of the row in float64. Nothing is sampled and nothing is fed back: it describes the file.
"""

from __future__ import annotations

import argparse
import json
import os
import sys



def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels serving uses; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to a page)")
    ap.add_argument("--page-size", type=int, default=None, help="tokens per cache page (default: the engine's)")
    ap.add_argument("--max-requests", type=int, default=8, help="most requests alive at once")
    ap.add_argument("--summary", default=None, help="also write a text line per wanted place to this file")
    args = ap.parse_args(argv)

    import torch
    from ..cache import DEFAULT_PAGE_SIZE
    from ..errors import EngineError
    from .build import build
    from .step import StepEntry
    from ..kernels import ops

    page = args.page_size or DEFAULT_PAGE_SIZE
    pool_tokens = -(-args.max_tokens // page) * page
    os.makedirs(args.out, exist_ok=True)
    try:
        built = build(args.model, dtype=args.dtype, kv_tokens=pool_tokens, max_batch_tokens=pool_tokens,
                      max_requests=args.max_requests, page_size=page, context=pool_tokens)
    except EngineError as e:
        print(f"trace_run: {e}", file=sys.stderr)
        return 1
    step_fn = built.step_fn
    summary = open(args.summary, "w", newline="\n") if args.summary else None

    def describe(step, entries, rows):
        import numpy as np
        r = 0
        for e in entries:
            for place in e.want:
                row = rows[r]
                order = np.lexsort((np.arange(row.size), -row))[:8]        # largest first, ties by lowest id
                wide = row.astype(np.float64)
                summary.write(f"step {step} id {e.request} place {place} argmax {int(order[0])} top "
                              + " ".join(f"{int(i)}:{row[i]:.6f}" for i in order)
                              + f" stats {float(wide.sum()):.6f} {float((wide * wide).sum()):.6f}\n")
                r += 1
        summary.flush()

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        try:
            obj = json.loads(line)
            step = obj["step"]
            entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in obj.get("entries", [])]
            if entries:
                logits = step_fn.step(entries)
                if logits is not None:
                    host = logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                    host.tofile(os.path.join(args.out, f"{step}.f32"))
                    if summary is not None:
                        describe(step, entries, host)
                else:
                    torch.cuda.current_stream().synchronize()
            if ops.gemm_tcgen05_status() != 0:
                raise EngineError("a tcgen05 matrix product gave up waiting on a barrier; its results are not valid")
            for req in obj.get("end", []):
                step_fn.end(req)
        except (EngineError, KeyError, ValueError, TypeError) as e:
            print(f"trace_run: step {line[:80]!r}: {type(e).__name__}: {e}", file=sys.stderr)
            return 1
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
