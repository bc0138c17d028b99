"""The plain implementation against dynalm-project/dynalm's own CPU Transformer.

tests/golden/<name>.logits.f32 were written by tests/golden/make_golden.py: the reference's
`Transformer::forward_batch` on its fp32 CPU device, whole prompt, logits at every position. The
weights are regenerated here from the same seed and must have the same checksum."""

import hashlib
import json
import os

import numpy as np
import pytest

from plain_llama import PlainLlama

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e", "f"])
def test_plain_matches_reference(name, tiny_folders):
    meta = json.load(open(os.path.join(GOLDEN, f"{name}.json")))
    folder = tiny_folders[name]
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        if hashlib.sha256(f.read()).hexdigest() != meta["weights_sha256"]:
            pytest.skip("this torch build draws other random weights than the one that made the golden files")
    golden = np.fromfile(os.path.join(GOLDEN, f"{name}.logits.f32"), dtype="<f4").reshape(meta["shape"])
    mine = PlainLlama(folder).logits(meta["prompt"])
    assert mine.shape == golden.shape
    err = np.abs(mine - golden).max()
    scale = np.abs(golden).max()
    assert err <= 2e-6 * max(1.0, scale), f"plain vs reference: max |diff| {err:.3g} at logit scale {scale:.3g}"
    assert (mine.argmax(-1) == golden.argmax(-1)).all()
