"""The command line on the CPU: what it answers before it needs a GPU (version, usage, refusals), and the
random-weights command, which writes a model folder that the loader reads back."""

import json
import os

from dynalm_b200.cli.main import main
from tiny_configs import TINY_B


def test_version_usage_and_unknown_command(capsys):
    assert main(["--version"]) == 0
    assert main(["version"]) == 0
    assert capsys.readouterr().out.count("dynalm_b200") == 2
    assert main([]) == 2                                    # nothing asked for: the usage text, as an error
    assert main(["--help"]) == 0
    err = capsys.readouterr().err
    assert "dynalm run" in err and "random-model" in err and "--solo-prefill-chunk" in err
    assert main(["serve"]) == 2                             # the server is not part of this engine
    assert "unknown command 'serve'" in capsys.readouterr().err


def test_run_refuses_what_it_does_not_offer(tmp_path, capsys):
    # the cache has the compute dtype: f16 is not offered, f32 only with the 32-bit mode
    assert main(["run", str(tmp_path), "--tokens", "1,2,3", "--kv", "f16"]) == 2
    assert "bf16" in capsys.readouterr().err
    assert main(["run", str(tmp_path), "--tokens", "1,2,3", "--kv", "f32"]) == 2
    assert "--mode exact" in capsys.readouterr().err
    # a folder without a model: one line, exit code 1 (with or without a GPU)
    assert main(["run", str(tmp_path / "nothing"), "--tokens", "1,2,3"]) == 1
    assert capsys.readouterr().err.startswith("dynalm: ")


def test_random_model_writes_a_folder_the_loader_reads(tmp_path, capsys):
    from dynalm_b200.weights import open_model_folder
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(TINY_B))
    one, two = tmp_path / "one", tmp_path / "two"
    assert main(["random-model", str(one), "--config", str(cfg), "--seed", "5", "--dtype", "f32"]) == 0
    assert main(["random-model", str(two), "--config", str(cfg), "--seed", "5", "--dtype", "f32"]) == 0
    assert capsys.readouterr().out.split() == [str(one), str(two)]
    assert sorted(os.listdir(one)) == ["config.json", "model.safetensors"]
    # the same seed gives the same bytes; the folder opens and names the architecture
    assert (one / "model.safetensors").read_bytes() == (two / "model.safetensors").read_bytes()
    folder = open_model_folder(str(one))
    assert folder.config.num_hidden_layers == TINY_B["num_hidden_layers"]
    assert len(folder.plan.layers) == TINY_B["num_hidden_layers"]
    folder.close()
