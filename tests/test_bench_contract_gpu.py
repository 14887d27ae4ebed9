"""bench.py prints one JSON line with the keys and shapes its contract names.  The run here is
cut to one layer and a few steps; the sizes of a layer stay those of the default run."""

import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    result = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                            timeout=600, cwd=ROOT)
    if result.returncode not in (0, 2):
        print(result.stderr[-3000:])           # shown by pytest when the test fails
    return result.returncode, result.stdout.strip().splitlines()


def test_bench_line_has_the_contract_keys():
    code, lines = run_bench("--layers", "1", "--steps", "4", "--warmup", "3")
    assert code == 0, lines
    assert len(lines) == 1, "exactly one line on standard output"
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "prefill", "roofline", "points", "clocks"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 4 and line["warmup"] == 3 and line["higher_is_better"] is True
    assert line["value"] > 0 and abs(line["value"] - line["config"]["global_batch"] * 1000.0 / line["ms_per_step"]) < 1e-6 * line["value"]
    config = line["config"]
    assert len(config) <= 20 and all(not isinstance(v, (dict, list)) for v in config.values()), "flat, at most 20 keys"
    assert config["layers"] == 1 and config["layers_full"] == 36, "a run with fewer layers names both numbers"
    assert set(line["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"}
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert set(line["prefill"]) >= {"value", "tokens", "ms", "frac"} and line["prefill"]["tokens"] == 2048
    assert line["roofline"]["bound"] == "hbm" and line["roofline"]["unit"] == "GB/s"
    assert abs(line["roofline"]["frac"] - line["roofline"]["achieved"] / line["roofline"]["peak"]) < 1e-9
    assert set(line["points"]) == {"decode_b1", "decode_b64"}
    assert set(line["workloads"]) == {"gen_1x512x32", "gen_4x2048x32", "gen_16x512x128"}
    assert all(v > 0 for v in line["workloads"].values())
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    assert line["gpu_launches"] > 0


def test_bench_refuses_more_than_one_gpu():
    code, lines = run_bench("--gpus", "2")
    assert code == 2 and len(lines) == 1


def test_reference_arm_prints_its_line_or_says_why_not():
    """With a copy of the reference's engine folder under baseline/_ref the arm runs the
    reference's own Engine on a one-layer model of the same sizes; without it, or if the
    reference does not start here, it says so in one line and exits 0."""
    code, lines = run_bench("--impl", "reference", "--layers", "1", "--steps", "4", "--warmup", "3", "--no-points")
    assert code == 0
    line = json.loads(lines[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and line["unavailable"]
    else:
        assert line["value"] > 0 and line["config"]["layers"] == 1 and line["config"]["layers_full"] == 36
        assert line["prefill"]["tokens"] == 2048 and line["e2e"]["value"] > 0
