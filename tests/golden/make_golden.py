"""Makes tests/golden/*.f32: logits of dynalm-project/dynalm's own CPU Transformer on tiny random models.

Run from the repository root on a machine that has the reference's source tree:

    python tests/golden/make_golden.py /path/to/dynalm

It configures a CPU-only build of the reference (native kernels, no server, no network), compiles
tests/golden/ref_harness.cpp against its two static libraries, writes each tiny model of
tests/tiny_configs.py with float32 random weights into a temporary folder, runs the harness on a fixed
prompt and stores `<name>.logits.f32` ([tokens, vocab] float32) and `<name>.json` (prompt, shapes,
a checksum of the weights) next to this file.
"""

import hashlib
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from tiny_configs import OPTIONAL_TENSORS, TINY  # noqa: E402
import dynalm_b200  # noqa: E402,F401
from dynalm_b200.weights import write_model_folder  # noqa: E402

PROMPT_LEN = {"a": 33, "b": 40, "c": 24, "d": 21, "e": 37, "f": 19, "g": 29}


def prompt_for(name: str, vocab: int):
    rng = np.random.RandomState({"a": 1, "b": 3, "c": 5, "d": 7, "e": 9, "f": 11, "g": 13}[name])
    return [int(t) for t in rng.randint(0, vocab, size=PROMPT_LEN[name])]


def weights_checksum(folder: str) -> str:
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def main():
    ref = os.path.abspath(sys.argv[1])
    build = os.environ.get("REF_BUILD", os.path.join(tempfile.gettempdir(), "refbuild"))
    subprocess.check_call(["cmake", "-S", ref, "-B", build, "-G", "Ninja", "-DDYNALM_NATIVE_ONLY=ON",
                           "-DENABLE_SERVER=OFF", "-DENABLE_BENCHMARKS=OFF"], stdout=subprocess.DEVNULL)
    subprocess.check_call(["ninja", "-C", build, "dynalm"], stdout=subprocess.DEVNULL)
    harness = os.path.join(build, "ref_harness")
    subprocess.check_call(["g++", "-std=c++20", "-O2", f"-I{ref}/dynalm/src", f"-I{ref}/dynacore/include",
                           f"-I{build}/dynalm/src/generated", os.path.join(HERE, "ref_harness.cpp"),
                           f"{build}/dynalm/src/libdynalm.a", f"{build}/dynacore/libdynacore.a",
                           "-lpthread", "-o", harness])
    for name, (cfg, seed) in TINY.items():
        with tempfile.TemporaryDirectory() as d:
            write_model_folder(d, cfg, seed, dtype=torch.float32, optional=OPTIONAL_TENSORS.get(name))
            toks = prompt_for(name, cfg["vocab_size"])
            out = os.path.join(HERE, f"{name}.logits.f32")
            print(subprocess.check_output([harness, d, out] + [str(t) for t in toks], text=True).strip())
            meta = {"config": cfg, "seed": seed, "prompt": toks, "shape": [len(toks), cfg["vocab_size"]],
                    "optional_tensors": OPTIONAL_TENSORS.get(name, []), "weights_sha256": weights_checksum(d)}
            with open(os.path.join(HERE, f"{name}.json"), "w") as f:
                json.dump(meta, f, indent=1)


if __name__ == "__main__":
    main()
