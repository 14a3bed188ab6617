"""The command line without a device: parsing, inspect, random folders, failure paths."""
import json

import pytest

import tiny_configs as tc
from cpp_minilamma_b200.cli import main, parse_ids


def test_parse_ids():
    assert parse_ids("5 17 3") == [5, 17, 3] and parse_ids("5,17, 3") == [5, 17, 3]
    with pytest.raises(SystemExit):
        parse_ids("hello")
    with pytest.raises(SystemExit):
        parse_ids("  ")


def test_random_then_inspect(tmp_path, capsys):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(tc.config("B").to_dict()))
    assert main(["random", str(tmp_path / "m"), "--config", str(cfg), "--seed", "4"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "architecture: LlamaForCausalLM" in out and "num_key_value_heads: 1" in out
    assert "tensor model.layers.2.mlp.down_proj.weight [192, 512] float32" in out
    assert "status=ok" in out
    params = int([line for line in out.splitlines() if line.startswith("parameters:")][0].split()[1])
    assert params == 257 * 192 + 3 * (2 * 192 + 192 * (192 + 32 + 32) + 192 * 192 + 3 * 192 * 512) + 192


def test_failures_exit_1_with_empty_stdout(tmp_path, capsys):
    assert main(["inspect", str(tmp_path / "nothing")]) == 1
    captured = capsys.readouterr()
    assert captured.out == "" and "config.json" in captured.err and "status=error" in captured.err
    assert main(["generate", str(tmp_path), "--backend", "cpu"]) == 1
    captured = capsys.readouterr()
    assert captured.out == "" and "CUDA path only" in captured.err
    assert main([]) == 1
    assert main(["generate", str(tmp_path), "--no-such-option"]) == 1
