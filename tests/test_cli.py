import pytest

from thing_htn_2026_b200 import cli


def test_shapes():
    assert cli.parse_shapes("1x5x4, 2x17x6") == [(1, 5, 4), (2, 17, 6)]
    for bad in ("", "2x3", "0x5x4", "axbxc".replace("a", "1").replace("b", "2").replace("c", "0")):
        with pytest.raises(SystemExit):
            cli.parse_shapes(bad)


def test_prompts_are_seeded_and_in_range():
    a, b = cli.make_prompt(3, 9, 300, 0), cli.make_prompt(3, 9, 300, 0)
    assert a == b and a != cli.make_prompt(3, 9, 300, 1)
    assert len(a) == 3 and all(len(r) == 9 and all(0 <= t < 300 for t in r) for r in a)


def test_help_runs(capsys):
    with pytest.raises(SystemExit) as info:
        cli.main(["--help"])
    assert info.value.code == 0
    assert "generate" in capsys.readouterr().out


def test_prompt_lens_and_named_configurations(tmp_path, capsys):
    import json
    import os
    from thing_htn_2026_b200.config import config_from_dict, named_config_json, named_configs
    assert cli.parse_lens("5, 9,16") == [5, 9, 16]
    for bad in ("", "3,x", "0,4"):
        with pytest.raises(SystemExit):
            cli.parse_lens(bad)
    prompts = cli.make_prompts_of([1, 23], 512, 7)
    assert [len(p) for p in prompts] == [1, 23] and prompts == cli.make_prompts_of([1, 23], 512, 7)
    assert {"tiny-a", "tiny-b", "qwen3-4b", "qwen3-8b", "qwen3-14b"} <= set(named_configs())
    for name in named_configs():
        config_from_dict(named_config_json(name))               # every preset passes the typed reader
    assert config_from_dict(named_config_json("qwen3-14b")).num_attention_heads == 40
    with pytest.raises(Exception, match="no configuration named"):
        named_config_json("qwen3-1t")
    # random-model runs without a device: a folder from a named configuration
    out = str(tmp_path / "m")
    assert cli.main(["random-model", "--random-config", "tiny-b", "--seed", "1", "--out", out, "--dtype", "fp32"]) == 0   # = float32
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(out, "config.json")))["num_key_value_heads"] == 1
    with pytest.raises(SystemExit):
        cli.main(["random-model", "--out", out])                # neither --config nor --random-config
