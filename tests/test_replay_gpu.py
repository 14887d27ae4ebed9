"""The engine against the plain implementation, in every way of cutting the work: each
request alone and whole; with its last 32 tokens one by one; in batches of unequal lengths
whose shorter requests end earlier, one batch after another so that slots and pages are
used again; long decoding; the first tokens of a sequence.  In 32-bit and in bfloat16, at
all tiny configurations."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import harness
import tiny

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = list(tiny.CONFIGS)


def make_requests(name, lengths, seed0=0):
    return {f"r{i}": tiny.tokens(name, n, seed0 + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(tiny_models, tmp_path, name, dtype):
    requests = make_requests(name, [5, 9, 16, 1, 23, 77, 130])
    got = harness.replay(tiny_models[name], dtype, harness.trace_whole(requests), str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], dtype, "whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(tiny_models, tmp_path, name, dtype):
    requests = make_requests(name, [40, 33, 97, 150], seed0=10)
    got = harness.replay(tiny_models[name], dtype, harness.trace_tail(requests, 32), str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], dtype, "tail")
    if dtype == "float32":
        # Every kernel of the 32-bit path computes a row from that row's own data in a fixed
        # order, so cutting changes nothing at all.
        whole = harness.replay(tiny_models[name], dtype, harness.trace_whole(requests), str(tmp_path / "w"))
        for r in requests:
            assert np.array_equal(got[r], whole[r]), f"{r}: float32 logits depend on the cutting"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_slot_reuse(tiny_models, tmp_path, name, dtype):
    lengths = [[30, 12, 70, 45], [9, 66, 20], [130, 5, 64, 65, 17]]
    prompts = [[5, 9, 16, 1], [1, 23, 20], [64, 3, 63, 65, 2]]
    batches, prompt_lens, requests = [], {}, {}
    for b, (ls, ps) in enumerate(zip(lengths, prompts)):
        batch = {}
        for i, (n, p) in enumerate(zip(ls, ps)):
            rid = f"b{b}r{i}"
            batch[rid] = tiny.tokens(name, n, 100 * b + i)
            prompt_lens[rid] = p
            requests[rid] = batch[rid]
        batches.append(batch)
    records = harness.trace_batches(batches, prompt_lens)
    got = harness.replay(tiny_models[name], dtype, records, str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], dtype, "batches")
    if dtype == "float32":
        alone = harness.replay(tiny_models[name], dtype, harness.trace_whole(requests), str(tmp_path / "w"))
        for r in requests:
            assert np.array_equal(got[r], alone[r]), f"{r}: float32 logits depend on the batch"


@pytest.mark.parametrize("policy", ["auto", "all"])
@pytest.mark.parametrize("name", NAMES)
def test_single_token_steps_through_the_streaming_product(tiny_models, tmp_path, name, policy, monkeypatch):
    """At the tiny sizes the few-row products would all go to the vendor library.  Here every
    product of a step of few rows (at most `ops.STREAM_MAX_ROWS`) is sent to this library's weight-streaming kernel
    (``all``: the gate-up product fused with SwiGLU as well), the head with float32 output
    included, and the logits are held to the same measure."""
    from thing_htn_2026_b200 import ops
    monkeypatch.setattr(ops, "STREAM_MIN_K", 0)
    monkeypatch.setattr(ops, "STREAM_MIN_N", 0)
    monkeypatch.setattr(ops, "STREAM_POLICY", policy)
    before = ops.launch_count
    requests = make_requests(name, [40, 33, 97], seed0=30)
    got = harness.replay(tiny_models[name], "bfloat16", harness.trace_tail(requests, 32), str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], "bfloat16", f"streaming products ({policy})")
    batches = [{k: requests[k] for k in ("r0", "r1")}, {"r2": requests["r2"]}]
    mixed = harness.replay(tiny_models[name], "bfloat16", harness.trace_batches(batches, {"r0": 7, "r1": 33, "r2": 64}),
                           str(tmp_path / "b"))
    harness.check_against_plain(mixed, requests, tiny_models[name], "bfloat16", f"streaming products, batches ({policy})")
    assert ops.launch_count > before


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "c", "d"])
def test_long_decoding(tiny_models, tmp_path, name, dtype):
    """A short prompt, then several hundred single-token steps across many pages."""
    requests = {"long": tiny.tokens(name, 300, 7), "short": tiny.tokens(name, 90, 8)}
    records = harness.trace_batches([requests], {"long": 3, "short": 2})
    got = harness.replay(tiny_models[name], dtype, records, str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(tiny_models, tmp_path, name, dtype):
    """A one-token prompt and the first few decoded tokens; several such requests at once."""
    requests = make_requests(name, [4, 1, 2, 6], seed0=50)
    records = harness.trace_batches([requests], {r: 1 for r in requests})
    got = harness.replay(tiny_models[name], dtype, records, str(tmp_path))
    harness.check_against_plain(got, requests, tiny_models[name], dtype, "first tokens")


def test_wanted_places_may_be_few_or_none(tiny_models, tmp_path):
    name = "b"
    toks = tiny.tokens(name, 20, 3)
    records = [
        {"step": 0, "entries": [{"id": "x", "tokens": toks[:10], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "x", "tokens": toks[10:], "want": [9, 0]}], "end": ["x"]},
    ]
    got = harness.replay(tiny_models[name], "float32", records, str(tmp_path))
    want = harness.plain_logits(tiny_models[name], toks, torch.float32)
    assert not os.path.exists(tmp_path / "0.f32")
    harness.assert_close_f32(got["x"], want[[19, 10]], "few places")


def test_trace_run_program(tiny_models, tmp_path):
    """The program itself: protocol on standard input and output, files, exit code."""
    name = "a"
    requests = make_requests(name, [12, 7])
    records = harness.trace_batches([requests], {"r0": 5, "r1": 3})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = "".join(json.dumps(r) + "\n" for r in records)
    result = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", tiny_models[name], "--dtype", "float32",
         "--out", str(tmp_path), "--max-tokens", str(harness.max_tokens_of(records))],
        input=text, capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr
    assert result.stdout.split("\n")[:len(records)] == [f"done {r['step']}" for r in records]
    first = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(8, tiny.CONFIGS[name]["vocab_size"])
    harness.assert_close_f32(first[:5], harness.plain_logits(tiny_models[name], requests["r0"], torch.float32)[:5],
                             "trace_run r0")
