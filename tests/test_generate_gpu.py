"""Generation through the Python entry point against the plain implementation: greedy
and temperature sampling, unequal prompts, stop tokens, sequences that end earlier,
several batches one after another, graphs on and off."""

import numpy as np
import pytest
import torch

import harness
import tiny
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def engine_for(model_dir, dtype, **kwargs):
    from thing_htn_2026_b200 import Engine
    return Engine(model_dir, dtype=dtype, **kwargs)


def collect(engine, prompts, n, **kwargs):
    """Runs generate; returns per-sequence token lists (None entries dropped) and the raw steps."""
    steps = list(engine.generate(prompts, n, **kwargs))
    tokens = [[s[i] for s in steps if s[i] is not None] for i in range(len(prompts))]
    return tokens, steps


def teacher_forced_margin(model_dir, dtype):
    """How far below the maximum a chosen logit may lie.  float32: rounding of sums only.
    bfloat16: four times the measured distance between the plain bfloat16 and float32
    logits (the reference accepts a fixed 2.0 at full size, tests/local_check.py:322-337)."""
    if dtype == "float32":
        return 1e-4
    probe = tiny.tokens_for_dir(model_dir, 40)
    noise = np.abs(harness.plain_logits(model_dir, probe, torch.bfloat16)
                   - harness.plain_logits(model_dir, probe, torch.float32)).max()
    return 4 * noise + 1e-3


def check_greedy(model_dir, dtype, prompt, emitted):
    """One teacher-forced plain forward over prompt + emitted tokens
    (tests/local_check.py:254-271): every emitted token is the argmax of the plain logits
    at its place, up to the margin."""
    full = list(prompt) + list(emitted)
    pdtype = torch.float32 if dtype == "float32" else torch.bfloat16
    logits = harness.plain_logits(model_dir, full, pdtype)
    margin = teacher_forced_margin(model_dir, dtype)
    for n, token in enumerate(emitted):
        row = logits[len(prompt) + n - 1]
        assert row[token] >= row.max() - margin, (
            f"token {n}: chose {token} ({row[token]:.5f}), plain argmax {row.argmax()} ({row.max():.5f})")
        if dtype == "float32":
            assert token == plain.greedy(row), f"token {n}: {token} != plain greedy {plain.greedy(row)}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_greedy_matches_plain(tiny_models, name, dtype):
    prompts = [tiny.tokens(name, n, 200 + i) for i, n in enumerate([5, 9, 16])]
    engine = engine_for(tiny_models[name], dtype)
    tokens, steps = collect(engine, prompts, 8)
    assert len(steps) == 8
    for step in steps:
        assert isinstance(step, list) and len(step) == 3
        assert all(type(t) is int and 0 <= t < tiny.CONFIGS[name]["vocab_size"] for t in step)
    for prompt, emitted in zip(prompts, tokens):
        check_greedy(tiny_models[name], dtype, prompt, emitted)
    assert engine.loop.decode_launches == 7       # never a step that cannot be needed


@pytest.mark.parametrize("name", ["a", "b"])
def test_temperature_sampling_matches_plain(tiny_models, name):
    """float32, temperature 0.7: each emitted token equals the plain Gumbel-max draw from the
    plain logits at its place, with the same (seed, stream, step)."""
    prompts = [tiny.tokens(name, n, 300 + i) for i, n in enumerate([1, 23])]
    engine = engine_for(tiny_models[name], "float32")
    tokens, _ = collect(engine, prompts, 12, temperature=0.7, seed=1234)
    differs_from_greedy = 0
    for i, (prompt, emitted) in enumerate(zip(prompts, tokens)):
        assert len(emitted) == 12
        logits = harness.plain_logits(tiny_models[name], list(prompt) + emitted, torch.float32)
        for n, token in enumerate(emitted):
            row = logits[len(prompt) + n - 1]
            assert token == plain.sample(row, 0.7, 1234, i, n), f"sequence {i} token {n}"
            differs_from_greedy += token != plain.greedy(row)
    assert differs_from_greedy > 0, "sampling never left the argmax: noise is not applied"


def test_sampling_does_not_depend_on_batch_mates(tiny_models):
    name = "b"
    prompts = [tiny.tokens(name, n, 400 + i) for i, n in enumerate([7, 3, 12])]
    engine = engine_for(tiny_models[name], "float32")
    together, _ = collect(engine, prompts, 10, temperature=[0.9, 0.0, 0.5], seed=77)
    from thing_htn_2026_b200.engine.generation import Request
    for i, prompt in enumerate(prompts):
        alone = engine.loop.generate_all([Request(prompt, 10, [0.9, 0.0, 0.5][i], 77, i)])[0]
        assert alone.tokens == together[i], f"sequence {i} sampled differently alone"


def test_stop_tokens_and_unequal_limits(tiny_models):
    name = "a"
    prompts = [tiny.tokens(name, n, 500 + i) for i, n in enumerate([6, 11, 2, 30])]
    engine = engine_for(tiny_models[name], "float32")
    free, _ = collect(engine, prompts, 12)
    stop = free[1][3]                       # sequence 1 shall stop at its 4th token
    limits = [12, 12, 5, 9]
    got, steps = collect(engine, prompts, limits, stop_token_ids=[stop])
    for i in range(4):
        want = free[i][:limits[i]]
        if stop in want:
            want = want[:want.index(stop) + 1]
        assert got[i] == want, f"sequence {i}"
    assert len(steps) == max(len(t) for t in got)
    for i in range(4):                      # after its end a sequence yields None, never a token
        tail = [s[i] for s in steps[len(got[i]):]]
        assert all(t is None for t in tail)
    engine.backend.cache.check()
    assert engine.backend.cache.book.open_slots() == [engine.backend._scratch_slot]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batches_one_after_another_reuse_slots(tiny_models, dtype):
    """A cache that holds two requests at a time, nine requests: successive
    batches on the same slots and pages give what each request gives alone."""
    name = "c"
    lengths = [5, 70, 20, 64, 1, 33, 90, 12, 7]
    prompts = [tiny.tokens(name, n, 600 + i) for i, n in enumerate(lengths)]
    small = engine_for(tiny_models[name], dtype, max_tokens=256, max_batch=2)
    done = small.generate_all(prompts, 6)
    assert len(small.loop.batches_run) >= 4
    small.backend.cache.check()
    assert [c.finish_reason for c in done] == ["length"] * 9
    if dtype == "float32":
        big = engine_for(tiny_models[name], dtype)
        for i, prompt in enumerate(prompts):
            alone, _ = collect(big, [prompt], 6)
            assert done[i].tokens == alone[0], f"request {i}"
    for prompt, c in zip(prompts, done):
        check_greedy(tiny_models[name], dtype, prompt, c.tokens)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_on_and_off_agree(tiny_models, dtype):
    name = "d"
    prompts = [tiny.tokens(name, n, 700 + i) for i, n in enumerate([3, 40, 65])]
    with_graphs, _ = collect(engine_for(tiny_models[name], dtype, graphs=True), prompts, 20,
                             temperature=[0.0, 0.8, 0.0], seed=5)
    without, _ = collect(engine_for(tiny_models[name], dtype, graphs=False, depth=1), prompts, 20,
                         temperature=[0.0, 0.8, 0.0], seed=5)
    assert with_graphs == without


def test_random_weights_engine_runs(tiny_models):
    from thing_htn_2026_b200 import Engine
    from thing_htn_2026_b200.config import config_from_dict
    config = config_from_dict(tiny.config_json("b"))
    engine = Engine.from_config(config, seed=3, dtype="float32", gain_std=0.1)
    tokens, steps = collect(engine, [[1, 2, 3], [4]], 5)
    assert len(steps) == 5 and all(len(t) == 5 for t in tokens)
    again, _ = collect(Engine.from_config(config, seed=3, dtype="float32", gain_std=0.1), [[1, 2, 3], [4]], 5)
    other, _ = collect(Engine.from_config(config, seed=4, dtype="float32", gain_std=0.1), [[1, 2, 3], [4]], 5)
    assert again == tokens, "the same seed draws other weights"
    assert other != tokens, "another seed draws the same weights"
    # the weights drawn on the device, written to a folder, give the same tokens through the loader
    # and are what the plain implementation needs to check them
    import tempfile
    from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
    from thing_htn_2026_b200.weights import random_tensors_on_device, write_safetensors
    import json, os
    drawn = random_tensors_on_device(tensor_specs_of_plan(config.plan()), 3, torch.float32, torch.device("cuda:0"),
                                     0.02, 0.1)
    with tempfile.TemporaryDirectory() as folder:
        write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.cpu() for k, v in drawn.items()})
        with open(os.path.join(folder, "config.json"), "w") as handle:
            json.dump(tiny.config_json("b"), handle)
        for prompt, emitted in zip([[1, 2, 3], [4]], tokens):
            check_greedy(folder, "float32", prompt, emitted)


def test_greedy_across_classes_of_context_length(tiny_models, monkeypatch):
    """A captured decode step is replayed only within its class of context length.  With the
    first class ending at 128 keys the longer sequence passes through three classes while it
    generates, the shorter one ends earlier, and every token still is the plain argmax."""
    from thing_htn_2026_b200 import ops
    monkeypatch.setattr(ops, "CONTEXT_CLASS_BASE", 128)
    name = "d"
    prompts = [tiny.tokens(name, n, 800 + i) for i, n in enumerate([100, 30])]
    engine = engine_for(tiny_models[name], "bfloat16")
    tokens, steps = collect(engine, prompts, [180, 40])
    assert [len(t) for t in tokens] == [180, 40]
    for prompt, emitted in zip(prompts, tokens):
        check_greedy(tiny_models[name], "bfloat16", prompt, emitted)
    assert {(2, 0), (2, 1), (1, 1), (1, 2)} <= {k[:2] for k in engine.backend.graphs}, sorted(engine.backend.graphs)
    engine.backend.cache.check()


def test_windowed_group_gives_pages_back_while_it_generates(tiny_models):
    """Generation maps pages step by step, so a layer group with a window of 70 keys holds a
    few pages per sequence however long the sequence grows, while the group that keeps all
    keys holds them all; the tokens are the plain argmax throughout."""
    name = "d"
    prompts = [tiny.tokens(name, n, 950 + i) for i, n in enumerate([10, 90])]
    engine = engine_for(tiny_models[name], "float32")
    book = None
    emitted = [[], []]
    most_windowed = 0
    for n, step in enumerate(engine.generate(prompts, 400)):
        book = engine.backend.cache.book
        windowed = [g for g, group in enumerate(book.groups) if group.window is not None]
        full = [g for g, group in enumerate(book.groups) if group.window is None]
        assert len(windowed) == 1 and len(full) == 1
        most_windowed = max(most_windowed, book.pages[windowed[0]].n_held)
        for seq, token in zip(emitted, step):
            seq.append(token)
    # 70 keys span at most three pages of 64, plus the page being written; two sequences, and the
    # backend's scratch slot holds one page
    assert most_windowed <= 2 * 4 + 1, most_windowed
    assert book.pages[full[0]].n_held == 1, "the batch has ended: only the scratch page is held"
    for prompt, tokens in zip(prompts, emitted):
        check_greedy(tiny_models[name], "float32", prompt, tokens)
    engine.backend.cache.check()
