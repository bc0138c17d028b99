"""The plain implementation against dynalm-project/dynalm's own CPU Transformer.

tests/golden/<name>.logits.f32 were written by tests/golden/make_golden.py: the reference's
`Transformer::forward_batch` on its fp32 CPU device, whole prompt, logits at every position. The
weights are regenerated here from the same seed by the package's own counter-based generator (integer
mixing and a Box-Muller transform, no library's random generator) and must have the same checksum: if
they do not, the test fails, since then nothing ties the plain implementation to the reference."""

import hashlib
import json
import os

import numpy as np
import pytest

from plain_llama import PlainLlama

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e", "f", "g"])
def test_plain_matches_reference(name, tiny_folders):
    meta = json.load(open(os.path.join(GOLDEN, f"{name}.json")))
    folder = tiny_folders[name]
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        assert hashlib.sha256(f.read()).hexdigest() == meta["weights_sha256"], \
            "the seeded weights are not the ones the golden logits were made from"
    golden = np.fromfile(os.path.join(GOLDEN, f"{name}.logits.f32"), dtype="<f4").reshape(meta["shape"])
    mine = PlainLlama(folder).logits(meta["prompt"])
    assert mine.shape == golden.shape
    err = np.abs(mine - golden).max()
    scale = np.abs(golden).max()
    assert err <= 2e-6 * max(1.0, scale), f"plain vs reference: max |diff| {err:.3g} at logit scale {scale:.3g}"
    assert (mine.argmax(-1) == golden.argmax(-1)).all()
