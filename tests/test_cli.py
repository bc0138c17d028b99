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


def test_config_file_environment_and_command_line_merge(tmp_path):
    """config file < DYNALM_* < command line, both file formats, unknown keys with their line."""
    import pytest
    from dynalm_b200.cli.config import merge_config, parse_config_text
    from dynalm_b200.cli.main import RUN_CONFIG_OPTIONS, _run_parser
    from dynalm_b200.errors import InvalidArgument, NotFound
    yaml = tmp_path / "config.yaml"
    yaml.write_text("# a comment\nruntime:\n  context_length: 2048   # tokens\n  batch_tokens: \"256\"\n"
                    "  threads: 8\nsampling:\n  temperature: 0.7\nserver:\n  port: 9000\nkv_cache:\n  dtype: bf16\n")
    env = {"DYNALM_CONFIG": str(yaml), "DYNALM_BATCH": "384", "DYNALM_MAX_TOKENS": "9"}
    merged = merge_config(["/m", "--tokens", "1,2", "--max-tokens", "5"], RUN_CONFIG_OPTIONS, env.get)
    # the server's port and the thread count are documented keys that `run` here has no option for: skipped
    assert merged == ["--ctx", "2048", "--batch", "256", "--temperature", "0.7", "--kv", "bf16", "--batch", "384",
                      "--max-tokens", "9", "/m", "--tokens", "1,2", "--max-tokens", "5"]
    args = _run_parser().parse_args(merged)
    assert (args.ctx, args.batch, args.temp, args.max_tokens, args.model) == ("2048", 384, 0.7, 5, "/m")
    # --config beats $DYNALM_CONFIG; the flat format; the model from the file
    flat = tmp_path / "flat.conf"
    flat.write_text("ctx = 512\nmodel = /from/file\nmode = exact\n")
    merged = merge_config(["--config", str(flat), "--prompt-len", "4"], RUN_CONFIG_OPTIONS, env.get)
    args = _run_parser().parse_args(merged)
    assert args.ctx == "512" and args.model_option == "/from/file" and args.mode == "exact" and args.batch == 384
    with pytest.raises(InvalidArgument, match=r"bad.yaml:2: unknown key 'runtime.speed'"):
        parse_config_text("runtime:\n  speed: 3\n", RUN_CONFIG_OPTIONS, "bad.yaml")
    with pytest.raises(InvalidArgument, match=r"f:1: unknown key 'port'"):
        parse_config_text("port = 1\n", RUN_CONFIG_OPTIONS, "f")
    with pytest.raises(InvalidArgument, match="lists"):
        parse_config_text("runtime:\n  threads: [1, 2]\n", RUN_CONFIG_OPTIONS, "f")
    with pytest.raises(NotFound):
        merge_config(["--config", str(tmp_path / "none.yaml")], RUN_CONFIG_OPTIONS, {}.get)
    with pytest.raises(InvalidArgument, match="--config needs"):
        merge_config(["--config"], RUN_CONFIG_OPTIONS, {}.get)
    # a file's error reaches the user as one line of `run`
    bad = tmp_path / "bad.yaml"
    bad.write_text("nonsense:\n  key: 1\n")
    assert main(["run", "/m", "--config", str(bad), "--tokens", "1"]) == 1


def test_log_levels_gate_the_package_lines(capsys):
    from dynalm_b200.utils import log
    before = log.level()
    try:
        assert main(["--log-level", "loud", "version"]) == 1
        assert "invalid log level 'loud'" in capsys.readouterr().err
        assert main(["--bogus", "version"]) == 1
        assert "unknown option '--bogus'" in capsys.readouterr().err
        for flags, shown in ((["-q"], {"error"}), ([], {"error", "warn", "info"}), (["-v"], {"error", "warn", "info", "debug"}),
                             (["--log-level", "off"], set()), (["--log-level=warn"], {"error", "warn"})):
            log.set_level("normal")
            assert main(flags + ["version"]) == 0
            capsys.readouterr()
            log.error("t", "error"), log.warn("t", "warn"), log.info("t", "info"), log.debug("t", "debug")
            assert set(capsys.readouterr().err.replace("[t] ", "").split()) == shown, flags
    finally:
        log.set_level(before)
