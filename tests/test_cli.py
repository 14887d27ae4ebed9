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
