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

QWEN3_4B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=2560,
    intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=5000000.0, tie_word_embeddings=True, max_position_embeddings=4096,
    hidden_act="silu", attention_bias=False, rope_scaling=None,
)
# Other layer sizes of the family, for measurements beside the default run (--sizes).
OTHER_SIZES = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, rope_theta=1000000.0, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                num_key_value_heads=8, rope_theta=1000000.0, tie_word_embeddings=False),
}
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
WORKLOADS = ((1, 512, 32), (4, 2048, 32), (16, 512, 128))     # AGENTS.md:56-60 of the reference
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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

    cfg = dict(QWEN3_4B)
    if args.sizes != "4b":
        cfg.update(OTHER_SIZES[args.sizes])
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
                if len(handles) > 4:
                    backend.fetch(handles.pop(0))
            end.record()
            torch.cuda.synchronize()
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

    # prefill of one 2,048-token prompt
    runner = backend.runner
    times = []
    n_prefills = max(3, min(args.warmup, 5)) + 3
    for rep in range(n_prefills):
        (slot,) = backend.cache.open(1)
        toks = prompts(1, PREFILL_TOKENS)[0]
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        profiled = args.profiler_range == "prefill" and rep == n_prefills - 1
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
    prefill_ms = statistics.median(times[3:])
    flops = prefill_flops(cfg, n_layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (prefill_ms * 1e-3), "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)}

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


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is not an installable package (pip: neither setup.py nor pyproject.toml "
                       "found), and its engine loads a checkpoint through a library loader that is not a "
                       "source here",
    }))
    return 0


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--sizes", default="4b", choices=["4b"] + sorted(OTHER_SIZES),
                        help="layer sizes of Qwen3-4B (the default run), -8B or -14B")
    parser.add_argument("--prompt-len", type=int, default=PROMPT, help="tokens of each prompt before the decode steps")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    parser.add_argument("--profiler-range", choices=["decode", "prefill"], default=None,
                        help="bracket the timed decode steps, or the last prefill, with cudaProfilerStart/Stop "
                             "(for ncu --profile-from-start off)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
