"""Model folders: the safetensors reader's refusals, the one error for wrong tensors, random weights."""

import json
import os
import struct

import pytest
import torch

import dynalm_b200
from dynalm_b200.errors import Corrupt, NotFound, Unsupported
from dynalm_b200.weights import (SafeTensorsFile, WeightMismatch, open_model_folder, random_tensors,
                                 write_model_folder, write_safetensors)
from dynalm_b200.registry import find_architecture
from tiny_configs import TINY_A, TINY_B


def _raw_file(path, header: dict, data: bytes = b"", hlen=None):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text) if hlen is None else hlen))
        f.write(text)
        f.write(data)


def test_round_trip_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16), "e": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafeTensorsFile(p)
    assert f.metadata == {"k": "v"}
    for n, v in t.items():
        got = f.tensor(n)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    # the file the reference's ecosystem reads: cross-check with the safetensors package when present
    try:
        from safetensors import safe_open
    except ImportError:
        return
    with safe_open(p, "pt") as g:
        for n, v in t.items():
            assert torch.equal(g.get_tensor(n), v)


def test_corrupt_headers(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    ok = {"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}
    cases = [
        (dict(hlen=1 << 40), "header length"),
        (dict(header={"w": {"dtype": "F32", "shape": [2, 2]}}), "lacks dtype, shape or data_offsets"),
        (dict(header={"w": {"dtype": "Q4", "shape": [2, 2], "data_offsets": [0, 16]}}), "unknown dtype"),
        (dict(header={"w": {"dtype": "F32", "shape": [1, 1, 1, 2, 2], "data_offsets": [0, 16]}}), "invalid shape"),
        (dict(header={"w": {"dtype": "F32", "shape": [2, -2], "data_offsets": [0, 16]}}), "invalid shape"),
        (dict(header={"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 64]}}), "outside the data"),
        (dict(header={"w": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 16]}}), "its shape needs 24"),
        (dict(header={"w": ok["w"], "v": {"dtype": "F32", "shape": [2], "data_offsets": [8, 16]}}), "overlap"),
    ]
    for kw, msg in cases:
        _raw_file(p, kw.get("header", ok), b"\0" * 16, kw.get("hlen"))
        with pytest.raises(Corrupt, match=msg):
            SafeTensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 5) + b"{{{{{")
    with pytest.raises(Corrupt, match="not valid JSON"):
        SafeTensorsFile(p)
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(Corrupt, match="too small"):
        SafeTensorsFile(p)
    _raw_file(p, {"w": {"dtype": "U8", "shape": [16], "data_offsets": [0, 16]}}, b"\0" * 16)
    with pytest.raises(Unsupported, match="cannot execute"):
        SafeTensorsFile(p).tensor("w")
    with pytest.raises(NotFound):
        SafeTensorsFile(str(tmp_path / "none.safetensors"))


def test_random_weights_are_seeded(tmp_path):
    arch = find_architecture(TINY_A)
    plan = arch.plan(arch.read_config(TINY_A))
    a, b, c = random_tensors(plan, 0), random_tensors(plan, 0), random_tensors(plan, 1)
    assert all(torch.equal(a[n], b[n]) for n in a) and any(not torch.equal(a[n], c[n]) for n in a)
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    nw = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(nw.mean().item() - 1.0) < 0.05 and 0.05 < nw.std().item() < 0.15
    # a tensor's values do not depend on which other tensors exist
    plan_b = find_architecture(TINY_B).plan(find_architecture(TINY_B).read_config(TINY_B))
    assert "lm_head.weight" in random_tensors(plan_b, 0) and "lm_head.weight" not in a


def test_folder_round_trip_and_tied_by_presence(tmp_path):
    d = str(tmp_path / "b")
    write_model_folder(d, TINY_B, 2, torch.float32)
    f = open_model_folder(d)
    assert f.architecture.name == "LlamaForCausalLM" and not f.plan.head.tied
    assert f.tensor("model.norm.weight").dtype == torch.float32
    # a file without lm_head is tied whatever config.json declares (the reference's adapter rule)
    t = {n: f.tensor(n).clone() for n in f.where if n != "lm_head.weight"}
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    assert open_model_folder(d).plan.head.tied


def test_one_error_lists_everything(tmp_path):
    d = str(tmp_path / "a")
    write_model_folder(d, TINY_A, 0, torch.float32)
    f = open_model_folder(d)
    t = {n: f.tensor(n).clone() for n in f.where}
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(192, 64)
    t["model.layers.7.mlp.extra.weight"] = torch.zeros(3)
    t["rotary.inv_freq"] = torch.zeros(8)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightMismatch) as e:
        open_model_folder(d)
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert sorted(err.unexpected) == ["model.layers.7.mlp.extra.weight", "rotary.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.layers.0.mlp.down_proj.weight",
                                                        "model.layers.0.self_attn.q_proj.weight"]
    msg = str(err)
    for needle in ("missing (2)", "unexpected (2)", "wrong shape (2)", "has [64, 32], expected [64, 64]"):
        assert needle in msg


def test_folder_errors(tmp_path):
    with pytest.raises(NotFound):
        open_model_folder(str(tmp_path / "nowhere"))
    d = tmp_path / "empty"
    d.mkdir()
    with pytest.raises(NotFound, match="config.json"):
        open_model_folder(str(d))
    (d / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(NotFound, match="no model.safetensors"):
        open_model_folder(str(d))
    (d / "config.json").write_text("[1, 2")
    with pytest.raises(Corrupt):
        open_model_folder(str(d))
    (d / "config.json").write_text(json.dumps(TINY_A))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../evil.safetensors"}}))
    with pytest.raises(Corrupt, match="plain file name"):
        open_model_folder(str(d))


def test_shards(tmp_path):
    d = str(tmp_path / "s")
    write_model_folder(d, TINY_A, 0, torch.float32)
    f = open_model_folder(d)
    names = sorted(f.where)
    t = {n: f.tensor(n).clone() for n in names}
    os.unlink(os.path.join(d, "model.safetensors"))
    half = len(names) // 2
    write_safetensors(os.path.join(d, "m-1.safetensors"), {n: t[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "m-2.safetensors"), {n: t[n] for n in names[half:]})
    wm = {n: ("m-1.safetensors" if i < half else "m-2.safetensors") for i, n in enumerate(names)}
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    g = open_model_folder(d)
    assert sorted(g.where) == names and torch.equal(g.tensor(names[-1]), t[names[-1]])
