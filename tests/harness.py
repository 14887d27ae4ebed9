"""Helpers of the GPU tests: traces (ways of cutting requests into steps), a replayer that
drives the library's own replay program in-process, and comparison with the plain
implementation."""

import os

import numpy as np
import torch

from plain import qwen3_plain as plain

PAGE = 64


def rounded(n):
    return -(-n // PAGE) * PAGE


# ----------------------------------------------------------------------------- traces
# A trace is a list of records {"step", "entries": [{"id", "tokens", "want"}], "end": []}.


def trace_whole(requests):
    """Each request alone, all its tokens in one step, logits at every place."""
    return [{"step": i, "entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}], "end": [name]}
            for i, (name, toks) in enumerate(requests.items())]


def trace_tail(requests, tail=32):
    """Each request alone: all but the last ``tail`` tokens in one step, then one by one."""
    records, step = [], 0
    for name, toks in requests.items():
        head = max(1, len(toks) - tail)
        records.append({"step": step, "entries": [{"id": name, "tokens": toks[:head], "want": list(range(head))}],
                        "end": []})
        step += 1
        for i in range(head, len(toks)):
            records.append({"step": step, "entries": [{"id": name, "tokens": [toks[i]], "want": [0]}],
                            "end": [name] if i == len(toks) - 1 else []})
            step += 1
        if head == len(toks):
            records[-1]["end"] = [name]
    return records


def trace_batches(batches, prompt_lens):
    """``batches``: list of dicts name -> tokens; the requests of a batch start together
    with prompts of ``prompt_lens[name]`` tokens, then go on one token each; a request ends
    when its tokens are used up, the others go on.  One batch after another."""
    records, step = [], 0
    for batch in batches:
        done = {name: prompt_lens[name] for name in batch}
        entries = [{"id": n, "tokens": t[:done[n]], "want": list(range(done[n]))} for n, t in batch.items()]
        ended = [n for n, t in batch.items() if done[n] == len(t)]
        records.append({"step": step, "entries": entries, "end": ended})
        step += 1
        live = [n for n in batch if n not in ended]
        while live:
            entries = [{"id": n, "tokens": [batch[n][done[n]]], "want": [0]} for n in live]
            for n in live:
                done[n] += 1
            ended = [n for n in live if done[n] == len(batch[n])]
            records.append({"step": step, "entries": entries, "end": ended})
            step += 1
            live = [n for n in live if n not in ended]
    return records


def max_tokens_of(records):
    """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held, peak = {}, 0
    for record in records:
        for e in record["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(rounded(n) for n in held.values()))
        for name in record["end"]:
            held.pop(name, None)
    return peak


# ----------------------------------------------------------------------------- replay


def replay(model_dir, dtype, records, out_dir, max_tokens=None):
    """Runs the records through the library's replayer; returns request -> [places, vocab]
    float32 logits in the order the places were asked for."""
    from thing_htn_2026_b200.engine.replay import Replayer
    os.makedirs(out_dir, exist_ok=True)
    with torch.inference_mode():
        replayer = Replayer(model_dir, dtype, max_tokens or max_tokens_of(records), out_dir)
        for record in records:
            replayer.run_step(record)
        replayer.cache.check()
        assert replayer.cache.tokens_held() == 0, "requests ended but tokens are still held"
    vocab = replayer.model.vocab_size
    out = {}
    for record in records:
        wanted = sum(len(e["want"]) for e in record["entries"])
        if not wanted:
            continue
        data = np.fromfile(os.path.join(out_dir, f"{record['step']}.f32"), dtype="<f4").reshape(wanted, vocab)
        row = 0
        for e in record["entries"]:
            n = len(e["want"])
            out.setdefault(e["id"], []).append(data[row:row + n])
            row += n
    return {name: np.concatenate(parts, axis=0) for name, parts in out.items()}


# ----------------------------------------------------------------------------- comparison

_plain_cache = {}


def plain_logits(model_dir, tokens, dtype):
    key = (model_dir, tuple(tokens), dtype)
    if key not in _plain_cache:
        _plain_cache[key] = plain.model_logits(model_dir, list(tokens), dtype).numpy()
    return _plain_cache[key]


# float32: the engine and the plain implementation differ only in the order of float32
# additions.  Logits of these models are O(1).
F32_ATOL = 3e-5


def assert_close_f32(got, want, what):
    err = np.abs(got - want).max()
    assert err <= F32_ATOL * max(1.0, np.abs(want).max()), f"{what}: float32 logits differ by {err:.3e}"


def assert_close_bf16(got, model_dir, tokens, what):
    """bfloat16: rounding points are the same in the engine and in the plain implementation,
    but a different order of float32 additions flips individual roundings, so the two
    differ by a fraction of bfloat16's own noise.  The noise is measured, not assumed: it is
    the distance of the plain bfloat16 logits from the plain float32 logits.  The engine
    must be as close to the plain bfloat16 result as that, and not farther from the
    float32 truth than twice that."""
    exact = plain_logits(model_dir, tokens, torch.float32)
    rounded_ = plain_logits(model_dir, tokens, torch.bfloat16)
    noise = np.abs(rounded_ - exact).max()
    err_plain = np.abs(got - rounded_).max()
    err_exact = np.abs(got - exact).max()
    assert err_plain <= noise + 1e-3, f"{what}: {err_plain:.3e} from plain bfloat16 (noise {noise:.3e})"
    assert err_exact <= 2 * noise + 1e-3, f"{what}: {err_exact:.3e} from float32 truth (noise {noise:.3e})"


def check_against_plain(results, requests, model_dir, dtype, what):
    for name, toks in requests.items():
        got = results[name]
        assert got.shape[0] == len(toks), f"{what} {name}: {got.shape[0]} places for {len(toks)} tokens"
        if dtype == "float32":
            assert_close_f32(got, plain_logits(model_dir, toks, torch.float32), f"{what} {name}")
        else:
            assert_close_bf16(got, model_dir, toks, f"{what} {name}")
