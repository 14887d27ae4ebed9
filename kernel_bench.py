"""Times the kernels of a decode step one by one at the Qwen3-4B layer sizes, each on cold
operands (the weights rotate through more copies than the L2 cache holds), with CUDA
events, and prints achieved GB/s beside the vendor library's product on the same shape.

    python kernel_bench.py [--batch 8] [--context 640] [--reps 20] [--sizes 4b|8b|14b]
"""

from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch  # noqa: E402

SIZES = {"4b": (2560, 9728, 151936, 32, 8, 128), "8b": (4096, 12288, 151936, 32, 8, 128),
         "14b": (5120, 17408, 151936, 40, 8, 128)}          # hidden, intermediate, vocab, q heads, kv heads, head size
H, I, V, NQ, NKV, D = SIZES["4b"]
L2_BYTES = 126 * 2 ** 20


def time_cold(make_call, n_variants, reps):
    """make_call(i) runs the op on operand set i; sets rotate so that each run reads cold data."""
    # The calls are recorded into one CUDA graph and replayed, so that the time is the
    # device's (back-to-back kernels, as in a decode step) and not the host's launch cost.
    for i in range(min(3, n_variants)):
        make_call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for r in range(reps):
            make_call(r % n_variants)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) / reps)
    return sorted(times)[len(times) // 2] * 1e3   # median per call, microseconds


def prefill_products(args):
    """The tcgen05 product against the vendor library at prompt sizes; the fused gate/up +
    SwiGLU against the library product followed by the SwiGLU kernel."""
    from thing_htn_2026_b200 import ops
    dev = "cuda:0"
    m = args.prefill_rows
    shapes = {"qkv": ((NQ + 2 * NKV) * D, H), "o": (H, NQ * D), "gate_up": (2 * I, H), "down": (H, I)}
    err = ops.new_error_word(dev)
    for name, (n, k) in shapes.items():
        copies = max(2, int(2 * L2_BYTES / (n * k * 2)) + 1)
        weights = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        flops = 2.0 * m * n * k
        own = time_cold(lambda i: ops.linear_tcgen05(x, weights[i], err), copies, args.reps)
        lib_us = time_cold(lambda i: torch.nn.functional.linear(x, weights[i]), copies, args.reps)
        entry = {"own_us": own, "own_tflops": flops / own / 1e6, "library_us": lib_us,
                 "library_tflops": flops / lib_us / 1e6}
        if name == "gate_up":
            fused = time_cold(lambda i: ops.linear_tcgen05(x, weights[i], err, swiglu=True), copies, args.reps)
            both = time_cold(lambda i: ops.swiglu(torch.nn.functional.linear(x, weights[i])), copies, args.reps)
            entry.update({"own_fused_swiglu_us": fused, "library_plus_swiglu_us": both})
        print(f"gemm_{name}_m{m}", json.dumps({k_: round(v, 2) for k_, v in entry.items()}))
        del weights
    # the kernels between the products, at their prompt sizes (inputs rotate through more than L2 holds)
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    copies = 4
    gus = [torch.randn(m, 2 * I, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    us = time_cold(lambda i: ops.swiglu(gus[i]), copies, args.reps)
    print(f"swiglu_m{m}", json.dumps({"own_us": round(us, 2), "gbs": round(m * 3 * I * 2 / us / 1e3, 1)}))
    del gus
    hs = [torch.randn(m, H, device=dev, dtype=torch.bfloat16) for _ in range(16)]
    ds = [torch.randn(m, H, device=dev, dtype=torch.bfloat16) for _ in range(16)]
    gain = torch.ones(H, device=dev, dtype=torch.bfloat16)
    us = time_cold(lambda i: ops.add_rmsnorm(hs[i], ds[i], gain, 1e-6), 16, args.reps)
    print(f"add_rmsnorm_m{m}", json.dumps({"own_us": round(us, 2), "gbs": round(m * 4 * H * 2 / us / 1e3, 1)}))
    del hs, ds
    cache = SequenceCache([KVSpec(NKV, D)] * copies, max_tokens=m + 64, dtype=torch.bfloat16, device=dev, max_slots=2)
    (slot,) = cache.open(1)
    cache.prepare([slot], [m])
    cu = torch.tensor([0, m], dtype=torch.int32, device=dev)
    rows = ops.step_rows(cu, torch.tensor([slot], dtype=torch.int32, device=dev), cache.seq_lens, m, m)
    rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": 1e6}), Runtime(torch.bfloat16, torch.device(dev), {}))
    rope.ensure(m + 64)
    qkvs = [torch.randn(m, (NQ + 2 * NKV) * D, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    views = [cache.kv_view(e) for e in range(copies)]
    us = time_cold(lambda i: ops.qk_norm_rope_cache(qkvs[i], gain[:D], gain[:D], 1e-6, rope.tables(), rows, views[i], NQ,
                                                     True, err), copies, args.reps)
    nbytes = m * ((NQ + 2 * NKV) * D * 2 + (NQ + 2 * NKV) * D * 2)
    print(f"qk_norm_rope_cache_m{m}", json.dumps({"own_us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)}))
    # causal attention of the whole prompt over the cache just written
    tile = ops.ROW_TILE()
    starts = list(range(0, m, tile))
    tiles = ops.RowTiles(torch.tensor(starts, dtype=torch.int32, device=dev),
                         torch.tensor([min(tile, m - r) for r in starts], dtype=torch.int32, device=dev),
                         len(starts), tile)
    qs = [torch.randn(m, NQ * D, device=dev, dtype=torch.bfloat16) for _ in range(copies)]
    for view in views:
        view.storage.normal_()
    us = time_cold(lambda i: ops.attention(qs[i], rows, views[i], NQ, D ** -0.5, None, err, tiles), copies, args.reps)
    flops = 4.0 * NQ * D * m * (m + 1) / 2
    print(f"attention_prefill_m{m}", json.dumps({"own_us": round(us, 2), "tflops": round(flops / us / 1e6, 1)}))
    assert int(err.item()) == 0


def results_print(results):
    for name, entry in results.items():
        print(name, json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in entry.items()}))


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=640)
    parser.add_argument("--reps", type=int, default=20)
    parser.add_argument("--prefill-rows", type=int, default=0,
                        help="instead of the decode kernels, time the many-row products at this row count")
    parser.add_argument("--only-attention", action="store_true", help="time the decode attention alone")
    parser.add_argument("--only-product", default="", help="time one few-row product alone: qkv, o, gate_up, down "
                        "or lm_head")
    parser.add_argument("--splits", default="", help="comma-separated split counts for the decode attention "
                        "(default: the library's own choice)")
    parser.add_argument("--sizes", default="4b", choices=sorted(SIZES), help="layer sizes of Qwen3-4B, -8B or -14B")
    args = parser.parse_args()
    global H, I, V, NQ, NKV, D
    H, I, V, NQ, NKV, D = SIZES[args.sizes]
    if args.prefill_rows:
        return prefill_products(args)
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    dev = "cuda:0"
    m = args.batch
    results = {}
    err = ops.new_error_word(dev)

    shapes = {"qkv": ((NQ + 2 * NKV) * D, H), "o": (H, NQ * D), "gate_up": (2 * I, H), "down": (H, I),
              "lm_head": (V, H)}
    if args.only_product:
        shapes = {args.only_product: shapes[args.only_product]}
    for name, (n, k) in ({} if args.only_attention else shapes).items():
        copies = max(2, int(2 * L2_BYTES / (n * k * 2)) + 1)
        weights = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        nbytes = n * k * 2
        entry = {"bytes": nbytes, "copies": copies}
        if ops.lib().thn_gemm_stream_supported(m, n, k):
            us = time_cold(lambda i: ops.linear_stream(x, weights[i], err=err), copies, args.reps)
            entry["stream_us"], entry["stream_gbs"] = us, nbytes / us / 1e3
        us = time_cold(lambda i: torch.nn.functional.linear(x, weights[i]), copies, args.reps)
        entry["library_us"], entry["library_gbs"] = us, nbytes / us / 1e3
        if name == "gate_up" and ops.lib().thn_gemm_stream_supported(m, n // 2, k):
            entry["stream_fused_swiglu_us"] = time_cold(
                lambda i: ops.linear_stream(x, weights[i], err=err, swiglu=True), copies, args.reps)
            entry["library_plus_swiglu_us"] = time_cold(
                lambda i: ops.swiglu(torch.nn.functional.linear(x, weights[i])), copies, args.reps)
        results[f"gemm_{name}_m{m}"] = entry
        del weights

    if args.only_product:
        return results_print(results)

    # decode attention over `context` cached tokens per sequence
    ctx = args.context
    caches = []
    n_copies = max(2, int(2 * L2_BYTES / (m * ctx * 2 * NKV * D * 2)) + 1)
    n_copies = min(n_copies, 64)
    cache = SequenceCache([KVSpec(NKV, D)] * n_copies, max_tokens=m * (ctx + 64), dtype=torch.bfloat16, device=dev,
                          max_slots=m + 1)
    slots = cache.open(m)
    cache.prepare(slots, [ctx] * m)
    cu = torch.arange(m + 1, dtype=torch.int32, device=dev) * ctx
    slots_dev = torch.tensor(slots, dtype=torch.int32, device=dev)
    rows = ops.step_rows(cu, slots_dev, cache.seq_lens, m * ctx, ctx)
    ops.advance(cache.seq_lens, slots_dev, cu)
    cache.commit(slots, [ctx] * m)
    cache.seq_lens -= 1                       # the step's own token sits at position ctx - 1
    cu1 = torch.arange(m + 1, dtype=torch.int32, device=dev)
    rows = ops.step_rows(cu1, slots_dev, cache.seq_lens, m, 1)
    q = torch.randn(m, NQ * D, device=dev, dtype=torch.bfloat16)
    views = [cache.kv_view(e) for e in range(n_copies)]
    for view in views:
        view.storage.normal_()
    nbytes = m * ctx * 2 * NKV * D * 2
    for splits in [int(s) for s in args.splits.split(",") if s] or [ops.decode_splits(m, NKV, dev, D, context=ctx)]:
        us = time_cold(lambda i: ops.attention_decode_bf16(q, rows, views[i], NQ, D ** -0.5, None, err,
                                                           n_splits=splits), n_copies, args.reps)
        results[f"attention_decode_b{m}_ctx{ctx}_splits{splits}"] = {"bytes": nbytes, "own_us": us,
                                                                     "own_gbs": nbytes / us / 1e3}
    if args.only_attention:
        return results_print(results)

    # the small kernels (latency-bound at this size)
    h = torch.randn(m, H, device=dev, dtype=torch.bfloat16)
    d = torch.randn(m, H, device=dev, dtype=torch.bfloat16)
    gain = torch.ones(H, device=dev, dtype=torch.bfloat16)
    results["add_rmsnorm"] = {"own_us": time_cold(lambda i: ops.add_rmsnorm(h, d, gain, 1e-6), 1, args.reps)}
    gu = torch.randn(m, 2 * I, device=dev, dtype=torch.bfloat16)
    results["swiglu"] = {"own_us": time_cold(lambda i: ops.swiglu(gu), 1, args.reps)}
    logits = torch.randn(m, V, device=dev, dtype=torch.float32)
    results["choose_tokens"] = {"own_us": time_cold(lambda i: ops.choose_tokens(logits), 1, args.reps)}
    assert int(err.item()) == 0, "a kernel reported an error"
    results_print(results)


if __name__ == "__main__":
    main()
