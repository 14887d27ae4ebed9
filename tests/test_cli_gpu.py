"""The command line end to end, as a user runs it: a model folder written by
``random-model``, tokens printed by ``generate``, and the same tokens from the Python
entry point on the same prompts (the reference drives its engine the same way from
tests/local_check.py:61-84)."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*args):
    done = subprocess.run([sys.executable, "-m", "thing_htn_2026_b200", *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return done.stdout.strip().splitlines()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_model_then_generate_prints_the_entry_points_tokens(tmp_path, dtype):
    from thing_htn_2026_b200 import Engine, cli
    folder = str(tmp_path / "model")
    assert run_cli("random-model", "--random-config", "tiny-b", "--seed", "1", "--out", folder, "--dtype", dtype,
                   "--gain-std", "0.1") == [folder]
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--shapes", "2x17x6,1x5x4",
                                                    "--seed", "0", "--dtype", dtype)]
    engine = Engine(folder, dtype=dtype)
    want = []
    for i, (b, s, n) in enumerate([(2, 17, 6), (1, 5, 4)]):
        steps = list(engine.generate(cli.make_prompt(b, s, engine.model.vocab_size, i), n))
        want += [[step[j] for step in steps] for j in range(b)]
    assert [p["tokens"] for p in printed] == want
    assert all(p["finish_reason"] == "length" for p in printed)

    # one batch of unequal prompts, sampled: --prompt-lens, --max-new-tokens, --temperature
    printed = [json.loads(line) for line in run_cli("generate", "--model", folder, "--prompt-lens", "1,23", "--seed", "7",
                                                    "--max-new-tokens", "12", "--temperature", "0.7", "--dtype", dtype)]
    prompts = cli.make_prompts_of([1, 23], engine.model.vocab_size, 7)
    steps = list(engine.generate(prompts, 12, temperature=0.7, seed=7))
    assert [p["tokens"] for p in printed] == [[step[j] for step in steps] for j in range(2)]


def test_generate_and_bench_from_a_named_configuration():
    printed = [json.loads(line) for line in run_cli("generate", "--random-config", "tiny-a", "--seed", "3",
                                                    "--prompt-lens", "5,9,16", "--max-new-tokens", "8")]
    assert len(printed) == 3 and all(len(p["tokens"]) == 8 for p in printed)
    lines = [json.loads(line) for line in run_cli("bench", "--random-config", "tiny-b", "--shapes", "2x16x8,1x40x5",
                                                  "--repeats", "1")]
    assert [line["shape"] for line in lines] == ["2x16x8", "1x40x5"]
    assert all(line["tok_per_s"] > 0 and line["ttft_ms"] > 0 for line in lines)
