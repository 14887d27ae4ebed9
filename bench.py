"""Decode and prefill throughput of the Qwen3-4B layer sizes with random bfloat16 weights
on one B200.  A "step" is one decode step of the whole batch.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second of K CUDA-graph decode steps
at the given batch (device time, CUDA events); ``e2e`` is the same through
``Engine.generate`` (host token lists in, host token lists out); ``prefill`` is one
2,048-token prompt; ``roofline`` compares the bytes a decode step has to read (every
weight once, the cache of the live requests) with the measured HBM copy bandwidth;
``points`` holds batch 1 and 64; ``workloads`` the reference's three public workloads
(batch x prompt x new tokens) as tokens per second of whole ``generate`` calls, prefill
included.  Only N=1 is supported.

``--impl reference`` runs the unmodified reference engine (a copy of its ``engine/`` folder
under ``baseline/_ref/``) through its own ``Engine(model_path).generate`` on the same
configuration, batch, prompt length and step counts, and prints the same line with
``"impl": "reference"``.  ``--workload 8b|14b`` runs the two larger workloads: batch 16 with
prompts of 64 to 2,048 tokens and 128 greedy steps at the Qwen3-8B sizes; batch 64 with
1,024-token prompts and 256 steps, half of the sequences sampling at temperature 0.8, at the
Qwen3-14B sizes.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZES = {"4b": "qwen3-4b", "8b": "qwen3-8b", "14b": "qwen3-14b"}     # named configurations of the package


def config_json(sizes):
    """The config.json of the package's named configuration (data under config/presets)."""
    with open(os.path.join(ROOT, "thing_htn_2026_b200", "config", "presets", SIZES[sizes] + ".json")) as handle:
        return json.load(handle)


CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
WORKLOADS = ((1, 512, 32), (4, 2048, 32), (16, 512, 128))     # AGENTS.md:56-60 of the reference
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
PREFILL_WARM, PREFILL_TIMED, PREFILL_MORE = 2, 3, 5
PREFILL_SETTLE_S = 3.0        # both arms repeat the prefill this long before the figure is taken


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as handle:
            data = json.load(handle)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if key in data:
                out[key] = float(data[key])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(cfg, n_layers):
    """Bytes and flops of the model at ``n_layers`` layers (bfloat16)."""
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Nq, Nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (Nq + 2 * Nkv) * D * H + Nq * D * H + 2 * I * H + I * H      # matrix elements
    gains = 2 * H + 2 * D
    weight_bytes = 2 * (n_layers * (per_layer + gains) + V * H + H)           # head read once (tied or not)
    kv_bytes_per_token = n_layers * 2 * Nkv * D * 2
    return {"matrix_per_layer": per_layer, "weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token}


def prefill_flops(cfg, n_layers, tokens):
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    Nq, D = cfg["num_attention_heads"], cfg["head_dim"]
    numbers = model_numbers(cfg, n_layers)
    gemm = 2.0 * tokens * n_layers * numbers["matrix_per_layer"] + 2.0 * V * H      # head on one row
    attention = n_layers * 2.0 * 2.0 * Nq * D * tokens * (tokens + 1) / 2            # QK and PV, causal
    return gemm + attention


def run_ours(args):
    import torch
    from thing_htn_2026_b200 import Engine, ops
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.engine.generation import Request
    from thing_htn_2026_b200.engine.step import StepEntry

    cfg = config_json(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    config = config_from_dict(cfg)
    peak = peaks()
    torch.manual_seed(0)
    biggest = max(args.batch, 64 if not args.no_points else args.batch)
    per_seq = args.prompt_len + max(args.steps + args.warmup, 64) + 64
    max_tokens = max(biggest * -(-per_seq // 64) * 64, 4096)
    if not args.no_points:
        max_tokens = max(max_tokens, max(b * -(-(p + n) // 64) * 64 for b, p, n in WORKLOADS))
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_batch=biggest)
    backend, vocab = engine.backend, cfg["vocab_size"]
    g = torch.Generator().manual_seed(0)

    def prompts(batch, length):
        return torch.randint(0, vocab, (batch, length), generator=g).tolist()

    def decode_device(batch, steps, warmup, sample_clocks=False):
        """K graph replays timed with CUDA events; returns ms per step and context seen."""
        requests = [Request(p, warmup + steps + 1, 0.0, 0, i) for i, p in enumerate(prompts(batch, args.prompt_len))]
        slots = backend.open_batch(requests)
        try:
            backend.fetch(backend.launch_prefill(slots, [r.tokens for r in requests]))
            for _ in range(warmup):
                backend.fetch(backend.launch_decode(slots))
            torch.cuda.synchronize()
            before = ops.launch_count
            sampler = ClockSampler() if sample_clocks else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if args.profiler_range == "decode" and sample_clocks:
                torch.cuda.profiler.start()
            start.record()
            handles = []
            for _ in range(steps):
                handles.append(backend.launch_decode(slots))
                if len(handles) > 3:
                    backend.fetch(handles.pop(0))
            end.record()
            torch.cuda.synchronize()
            for handle in handles:
                backend.fetch(handle)
            if args.profiler_range == "decode" and sample_clocks:
                torch.cuda.profiler.stop()
            clocks = sampler.stop() if sampler else None
            ms = start.elapsed_time(end) / steps
            ctx_mean = args.prompt_len + warmup + (steps - 1) / 2.0
            return ms, ctx_mean, clocks, ops.launch_count - before
        finally:
            backend.close_batch(slots)

    # graphs are captured (and their kernels counted) during warm-up
    ops.launch_count = 0
    ms, ctx_mean, clocks, host_calls = decode_device(args.batch, args.steps, max(args.warmup, 3), sample_clocks=True)
    value = args.batch * 1000.0 / ms
    numbers = model_numbers(cfg, n_layers)
    step_bytes = numbers["weight_bytes"] + args.batch * 2 * cfg["hidden_size"] \
        + args.batch * ctx_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # kernels of this library per decode step: count one eager run of the program
    eager_before = ops.launch_count
    probe = [Request(p, 3, 0.0, 0, i) for i, p in enumerate(prompts(args.batch, 8))]
    slots = backend.open_batch(probe)
    backend.fetch(backend.launch_prefill(slots, [r.tokens for r in probe]))
    backend._set_composition(slots)
    mark = ops.launch_count
    backend._decode_program(args.batch, ops.context_class(16)[1])
    backend.cache.commit(list(slots), [1] * args.batch)
    own_per_step = ops.launch_count - mark
    torch.cuda.synchronize()
    backend.close_batch(slots)

    # end to end through the public entry point
    e2e_prompts = prompts(args.batch, args.prompt_len)
    n_new = args.steps + 1
    list(engine.generate(e2e_prompts, 4))                   # warm: graphs for this batch exist already
    torch.cuda.synchronize()
    uploaded_before = backend.runner.uploaded_bytes
    t0 = time.perf_counter()
    t_first = None
    count = 0
    for step_tokens in engine.generate(e2e_prompts, n_new):
        if t_first is None:
            t_first = time.perf_counter()
        count += 1
    t1 = time.perf_counter()
    assert count == n_new
    e2e_uploaded = backend.runner.uploaded_bytes - uploaded_before
    e2e_decode = args.batch * (n_new - 1) / (t1 - t_first)
    e2e_total = args.batch * n_new / (t1 - t0)

    # prefill of one 2,048-token prompt, the same protocol in both arms.  How fast a GPU under its
    # power cap runs a step like this depends on how warm the minutes before have left it (the arm
    # that runs first on a fresh GPU measured 14.1 ms in its first steps, the other arm 15.3-15.6,
    # whichever engine it was), so the figure is taken where that history has faded: the step is
    # repeated for PREFILL_SETTLE_S seconds and the median of the last five counts.  The median of
    # PREFILL_TIMED steps after the first PREFILL_WARM is kept beside it as `ms_first`.
    runner = backend.runner
    times = []
    settle_started = time.perf_counter()
    rep = 0
    while rep < PREFILL_WARM + PREFILL_TIMED + PREFILL_MORE or time.perf_counter() - settle_started < PREFILL_SETTLE_S:
        (slot,) = backend.cache.open(1)
        toks = prompts(1, PREFILL_TOKENS)[0]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        profiled = args.profiler_range == "prefill" and rep == PREFILL_WARM + PREFILL_TIMED - 1
        if profiled:
            torch.cuda.profiler.start()
        start.record()
        logits = runner.step([StepEntry(slot, toks, (PREFILL_TOKENS - 1,))], check=False)
        end.record()
        torch.cuda.synchronize()
        if profiled:
            torch.cuda.profiler.stop()
        times.append(start.elapsed_time(end))
        backend.cache.close([slot])
        rep += 1
        if args.profiler_range == "prefill" and rep >= PREFILL_WARM + PREFILL_TIMED:
            break                                           # a profiled run needs no more than its one step
    first_ms = statistics.median(times[PREFILL_WARM:PREFILL_WARM + PREFILL_TIMED])
    prefill_ms = statistics.median(times[-5:])
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak.get("bf16_tflops_sustained", peak["bf16_tflops"]) * 1e12),
               "peak_tflops": peak.get("bf16_tflops_sustained", peak["bf16_tflops"]),
               "frac_burst": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
               "ms_first": first_ms, "steps": len(times),
               "note": f"median of the last 5 of {len(times)} steps in a row ({PREFILL_SETTLE_S:.0f} s), so frac is against the "
                       f"peak of a seconds-long loop under the power cap (peak_tflops) and frac_burst against the burst "
                       f"peak; ms_first: median of {PREFILL_TIMED} steps after {PREFILL_WARM}"}

    points = {}
    if not args.no_points:
        for batch in (1, 64):
            pms, _, _, _ = decode_device(batch, min(args.steps, 64), 3)
            points[f"decode_b{batch}"] = batch * 1000.0 / pms

    # The reference's public workloads (batch x prompt x new tokens), by its own definition of
    # throughput: batch * new tokens / time of the whole call, prefill included.
    workloads = {}
    if not args.no_points:
        for batch, prompt_len, n_out in WORKLOADS:
            best = None
            for attempt in range(3):                             # the first call captures the graphs
                w_prompts = prompts(batch, prompt_len)
                torch.cuda.synchronize()
                w0 = time.perf_counter()
                produced = sum(1 for _ in engine.generate(w_prompts, n_out))
                w1 = time.perf_counter()
                assert produced == n_out
                if attempt:
                    best = min(best or w1 - w0, w1 - w0)
            workloads[f"gen_{batch}x{prompt_len}x{n_out}"] = batch * n_out / best

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": f"Qwen3-{args.sizes.upper()} layer sizes", "layers": n_layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": max(CONTEXT, args.prompt_len + args.steps + max(args.warmup, 3) + 1), "prompt_len": args.prompt_len,
            "context_mean": ctx_mean, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads all weights)", "graphs": backend.use_graphs,
            "peaks": peak["source"],
        },
        "e2e": {"value": e2e_decode, "unit": "tok/s", "with_prefill": e2e_total,
                "h2d_bytes_per_step": e2e_uploaded / n_new,
                "d2h_bytes_per_step": args.batch * 4,
                "note": "whole generate() call: prompts from pinned host memory, one token per sequence "
                        "read back every step; value counts the decode steps, with_prefill the whole call"},
        "gpu_launches": own_per_step * args.steps,
        "own_kernels_per_step": own_per_step,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "workloads": workloads,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- the larger workloads

LARGE_WORKLOADS = {
    # sizes, batch, (shortest, longest) prompt, decode steps, temperature of every second sequence
    "8b": ("8b", 16, (64, 2048), 128, 0.0),
    "14b": ("14b", 64, (1024, 1024), 256, 0.8),
}


def run_workload(args):
    """One of the two larger workloads, prefill and decode timed on the device."""
    import torch
    from thing_htn_2026_b200 import Engine
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.engine.generation import Request

    sizes, batch, (shortest, longest), steps, temperature = LARGE_WORKLOADS[args.workload]
    steps = args.steps if args.steps_given else steps
    cfg = config_json(sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    peak = peaks()
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(shortest, longest + 1, (batch,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    warmup = max(args.warmup, 3)
    n_new = warmup + steps + 1
    max_tokens = sum(-(-(n + n_new) // 64) * 64 for n in lens)
    engine = Engine.from_config(config_from_dict(cfg), seed=0, dtype="bfloat16", max_tokens=max_tokens, max_batch=batch)
    backend = engine.backend
    requests = [Request(p, n_new, temperature if i % 2 else 0.0, 1234, i) for i, p in enumerate(prompts)]

    def one_run(timed):
        slots = backend.open_batch(requests)
        try:
            start, mid, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            torch.cuda.synchronize()
            start.record()
            first = backend.launch_prefill(slots, prompts)
            mid.record()
            backend.fetch(first)
            for _ in range(warmup):
                backend.fetch(backend.launch_decode(slots))
            torch.cuda.synchronize()
            sampler = ClockSampler() if timed else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            handles = []
            for _ in range(steps):
                handles.append(backend.launch_decode(slots))
                if len(handles) > 3:
                    backend.fetch(handles.pop(0))
            t1.record()
            torch.cuda.synchronize()
            for h in handles:
                backend.fetch(h)
            clocks = sampler.stop() if sampler else None
            return start.elapsed_time(mid), t0.elapsed_time(t1) / steps, clocks
        finally:
            backend.close_batch(slots)

    one_run(False)                                   # captures the graphs, settles the allocator
    prefill_ms, ms, clocks = one_run(True)
    numbers = model_numbers(cfg, n_layers)
    context_mean = sum(lens) / batch + warmup + (steps - 1) / 2.0
    step_bytes = numbers["weight_bytes"] + batch * context_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = sum(prefill_flops(cfg, n_layers, n) for n in lens)
    line = {
        "metric": f"decode tok/s at batch {batch} (Qwen3-{sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": batch * 1000.0 / ms, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random-init weights, seeded uniform-random token ids", "impl": "ours",
        "config": {"model": f"Qwen3-{sizes.upper()} layer sizes", "workload": args.workload, "layers": n_layers,
                   "layers_full": full_layers, "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": bool(cfg["tie_word_embeddings"]), "global_batch": batch, "prompt_min": min(lens),
                   "prompt_max": max(lens), "prompt_tokens": sum(lens), "context_mean": context_mean,
                   "sampled_sequences": sum(1 for r in requests if r.temperature > 0), "temperature": temperature,
                   "parallelism": "single GPU", "peaks": peak["source"]},
        "prefill": {"value": sum(lens) / (prefill_ms * 1e-3), "tokens": sum(lens), "ms": prefill_ms,
                    "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------- the reference arm

REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def run_reference(args):
    """The unmodified reference: its ``engine/`` folder as copied to ``baseline/_ref/engine``,
    built by its own ``Engine(model_path)`` on a random Qwen3-4B-size folder and driven through
    its own ``generate(input_ids, max_new_tokens)``.  Nothing of this repository's package is
    imported into this process: the folder is written by a child process."""
    engine_dir = os.path.join(REF_DIR, "engine")
    if not os.path.isfile(os.path.join(engine_dir, "engine.py")):
        return unavailable(f"no copy of the reference's engine/ folder under baseline/_ref (looked for "
                           f"{os.path.relpath(engine_dir, ROOT)}/engine.py)")
    cfg = config_json(args.sizes)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    n_layers = cfg["num_hidden_layers"]
    warmup = max(args.warmup, 3)
    folder = tempfile.mkdtemp(prefix="thn_reference_model_")
    try:
        made = subprocess.run(
            [sys.executable, "-m", "thing_htn_2026_b200", "random-model", "--random-config", SIZES[args.sizes],
             "--layers", str(args.layers), "--seed", "0", "--dtype", "bfloat16", "--device", "cuda:0", "--out", folder],
            cwd=ROOT, capture_output=True, text=True)
        if made.returncode != 0:
            return unavailable(f"could not write the random model folder: {made.stderr.strip()[-300:]}")
        try:
            sys.path.insert(0, engine_dir)
            import torch
            import engine as reference_engine              # baseline/_ref/engine/engine.py
            ref = reference_engine.Engine(folder)
        except Exception as error:  # noqa: BLE001 - whatever stops the reference from starting is the answer
            return unavailable(f"the reference engine did not start: {type(error).__name__}: {error}")
        return time_reference(args, ref, torch, cfg, n_layers, full_layers, warmup)
    finally:
        import shutil
        shutil.rmtree(folder, ignore_errors=True)


def time_reference(args, ref, torch, cfg, n_layers, full_layers, warmup):
    peak = peaks()
    vocab = cfg["vocab_size"]
    g = torch.Generator().manual_seed(0)

    def prompts(batch, length):
        return torch.randint(0, vocab, (batch, length), generator=g).tolist()

    def decode(batch, steps, sample_clocks=False):
        """Wall time between the yields of ``generate`` after ``warmup`` decode steps: host token
        lists in, host token lists out, as its caller sees them."""
        n_new = 1 + warmup + steps
        list(ref.generate(prompts(batch, args.prompt_len), n_new))          # its per-shape preparation and graph capture
        sampler = ClockSampler() if sample_clocks else None
        ids = prompts(batch, args.prompt_len)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        stamps = []
        for i, tokens in enumerate(ref.generate(ids, n_new)):
            stamps.append(time.perf_counter())
            if i == warmup and sampler:
                sampler.start()
        clocks = sampler.stop() if sampler else None
        assert len(stamps) == n_new and len(tokens) == batch
        seconds = stamps[-1] - stamps[warmup]
        return 1e3 * seconds / steps, 1e3 * (stamps[0] - t0), clocks, batch * n_new / (stamps[-1] - t0)

    started = time.perf_counter()
    ms, _, clocks, with_prefill = decode(args.batch, args.steps, sample_clocks=True)
    value = args.batch * 1000.0 / ms
    numbers = model_numbers(cfg, n_layers)
    ctx_mean = args.prompt_len + warmup + (args.steps - 1) / 2.0
    step_bytes = numbers["weight_bytes"] + args.batch * 2 * cfg["hidden_size"] \
        + args.batch * ctx_mean * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9

    # time to the first token of one 2,048-token prompt, by the other arm's protocol: the calls
    # are repeated for PREFILL_SETTLE_S seconds and the median of the last five counts; the median
    # of PREFILL_TIMED calls after the first PREFILL_WARM (the first of them also prepares the
    # reference's state for this shape) is kept as `ms_first`.
    times = []
    list(ref.generate(prompts(1, PREFILL_TOKENS), 2))
    settle_started = time.perf_counter()
    rep = 1
    while rep < PREFILL_WARM + PREFILL_TIMED + PREFILL_MORE or time.perf_counter() - settle_started < PREFILL_SETTLE_S:
        ids = prompts(1, PREFILL_TOKENS)
        torch.cuda.synchronize()
        profiled = args.profiler_range == "prefill" and rep == PREFILL_WARM + PREFILL_TIMED - 1
        if profiled:
            torch.cuda.profiler.start()
        t0 = time.perf_counter()
        for tokens in ref.generate(ids, 1):
            times.append(1e3 * (time.perf_counter() - t0))
        if profiled:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        rep += 1
        if args.profiler_range == "prefill" and rep >= PREFILL_WARM + PREFILL_TIMED:
            break
    first_ms = statistics.median(times[PREFILL_WARM - 1:PREFILL_WARM - 1 + PREFILL_TIMED])
    prefill_ms = statistics.median(times[-5:])
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)

    points = {}
    if not args.no_points:
        for batch in (1, 64):
            if time.perf_counter() - started > 420:          # each new shape costs the reference a warm-up
                break
            pms, _, _, _ = decode(batch, min(args.steps, 64))
            points[f"decode_b{batch}"] = batch * 1000.0 / pms

    # Its own public workloads (batch x prompt x new tokens), by its own definition of throughput:
    # batch * new tokens / time of the whole call, prefill included; the best of two calls after one.
    workloads = {}
    if not args.no_points:
        for batch, prompt_len, n_out in WORKLOADS:
            if time.perf_counter() - started > 600:
                break
            best = None
            for attempt in range(3):
                w_prompts = prompts(batch, prompt_len)
                torch.cuda.synchronize()
                w0 = time.perf_counter()
                produced = sum(1 for _ in ref.generate(w_prompts, n_out))
                w1 = time.perf_counter()
                assert produced == n_out
                if attempt:
                    best = min(best or w1 - w0, w1 - w0)
            workloads[f"gen_{batch}x{prompt_len}x{n_out}"] = batch * n_out / best

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.sizes.upper()} layer sizes, random bf16 weights, 1 B200)",
        "value": value, "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random-init weights, seeded uniform-random token ids",
        "impl": "reference",
        "config": {
            "model": f"Qwen3-{args.sizes.upper()} layer sizes", "layers": n_layers, "layers_full": full_layers,
            "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "tied": bool(cfg["tie_word_embeddings"]),
            "global_batch": args.batch, "seq_len": max(CONTEXT, args.prompt_len + args.steps + warmup + 1),
            "prompt_len": args.prompt_len, "context_mean": ctx_mean, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (a step reads all weights)", "graphs": bool(getattr(ref, "use_graphs", False)),
            "peaks": peak["source"],
        },
        "e2e": {"value": value, "unit": "tok/s", "with_prefill": with_prefill,
                "h2d_bytes_per_step": args.batch * args.prompt_len * 8 / (1 + warmup + args.steps),
                "d2h_bytes_per_step": args.batch * 8,
                "note": "the reference has one public call, generate(): value and e2e are the same wall-clock "
                        "measurement between its yields (prompt ids uploaded once as int64, one int64 token per "
                        "sequence read back every step)"},
        "gpu_launches": None,
        "triton": bool(getattr(ref, "use_triton", False)),
        "ops": {name: getattr(fn, "__module__", "?").split(".")[-1] for name, fn in getattr(ref, "ops", {}).items()},
        "prefill": {"value": PREFILL_TOKENS / (prefill_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
                    "frac": flops / (prefill_ms * 1e-3) / (peak.get("bf16_tflops_sustained", peak["bf16_tflops"]) * 1e12),
                    "peak_tflops": peak.get("bf16_tflops_sustained", peak["bf16_tflops"]),
                    "frac_burst": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12),
                    "ms_first": first_ms, "steps": len(times),
                    "note": f"time to the first token of generate(), host to host; median of the last 5 of {len(times)} "
                            f"calls in a row ({PREFILL_SETTLE_S:.0f} s); ms_first: median of {PREFILL_TIMED} calls after "
                            f"{PREFILL_WARM}"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "bytes_per_step": step_bytes},
        "points": points,
        "workloads": workloads,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="timed decode steps (default 256)")
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--sizes", default="4b", choices=sorted(SIZES),
                        help="layer sizes of Qwen3-4B (the default run), -8B or -14B")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the decode steps")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    parser.add_argument("--profiler-range", choices=["decode", "prefill"], default=None,
                        help="bracket the timed decode steps, or the last prefill, with cudaProfilerStart/Stop "
                             "(for ncu --profile-from-start off)")
    parser.add_argument("--workload", choices=sorted(LARGE_WORKLOADS), default=None,
                        help="one of the two larger workloads instead of the default run")
    args = parser.parse_args()
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 256
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.workload:
        return run_workload(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
