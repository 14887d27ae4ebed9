"""The schedules that the tiny models never reach and that, without these tests, only the
measurement program would run: decode attention with dozens of (sequence, kv head) pairs
(one block per pair, fewer tile buffers, a second pass), generation's captured decode
program at the layer sizes of Qwen3-4B, the head product at its full width, and the device
error word's bits."""

import numpy as np
import pytest
import torch

import harness
import test_kernels_gpu as kernels
from test_real_sizes_gpu import CONFIG, model_dir, requests  # noqa: F401  (model_dir is a fixture)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from thing_htn_2026_b200 import ops as o
    return o


def spread_lengths(n_seqs, longest=700):
    """1 ... longest, spread over the sequences and shuffled: one key, page edges, many pages."""
    g = torch.Generator().manual_seed(n_seqs)
    base = [1 + (i * (longest - 1)) // max(1, n_seqs - 1) for i in range(n_seqs)]
    for i, special in enumerate([64, 65, 128, 129]):
        base[3 + 5 * i] = special
    order = torch.randperm(n_seqs, generator=g).tolist()
    return [base[i] for i in order]


# ----------------------------------------------------------------------------- decode attention, many pairs

@pytest.fixture
def streaming_always():
    """Every unsplit single-token step goes to the streaming kernel, however few its pairs."""
    o = ops()
    o.lib().thn_set_decode_stream(2, 3)
    yield
    o.lib().thn_set_decode_stream(1, 3)



seen_variants = {}


@pytest.mark.parametrize("splits", ["", "1"])
@pytest.mark.parametrize("n_seqs", [40, 48, 56, 64])
def test_decode_attention_with_many_pairs(n_seqs, splits, streaming_always):
    """32 query heads on 8 kv heads of 128 (the Qwen3-4B attention) for 40 to 64 sequences:
    320 to 512 (sequence, kv head) pairs, more than fit the GPU as clusters, through the
    streaming kernel (which by itself takes the steps that would need a second pass: 56 and 64
    sequences here)."""
    o = ops()
    dtype = torch.bfloat16
    lengths = spread_lengths(n_seqs)
    got, want = kernels.attention_case("decode" + splits, dtype, 32, 8, 128, lengths, [1] * n_seqs, None)
    kernels.close(got, want, dtype, f"decode attention, {n_seqs} sequences, splits {splits or 'auto'}")
    variant = o.lib().thn_attention_decode_last_variant()
    assert variant % 10 == 2, "hundreds of pairs, one split: the streaming kernel's step"


@pytest.mark.parametrize("stages", [3, 6])
@pytest.mark.parametrize("n_seqs", [40, 48, 56, 64])
def test_decode_attention_with_many_pairs_one_block_per_pair(n_seqs, stages):
    """The same steps with the streaming kernel switched off (one block per pair with six,
    three or two tile buffers, at the top a second pass) and with its deeper ring of tile
    buffers."""
    o = ops()
    dtype = torch.bfloat16
    lengths = spread_lengths(n_seqs)
    try:
        o.lib().thn_set_decode_stream(0 if stages == 3 else 2, stages)       # off; or always, with the deeper ring
        got, want = kernels.attention_case("decode", dtype, 32, 8, 128, lengths, [1] * n_seqs, None)
        variant = o.lib().thn_attention_decode_last_variant()
    finally:
        o.lib().thn_set_decode_stream(1, 3)
    kernels.close(got, want, dtype, f"decode attention, {n_seqs} sequences")
    if stages == 3:
        assert variant % 10 == 0, "hundreds of pairs were given to clusters"
        seen_variants[n_seqs] = variant // 10
    else:
        assert variant == 62


def test_decode_attention_many_pairs_took_every_branch():
    """The four batch sizes above reach the one-block-per-pair variants with two and three tile
    buffers (which of them at which size depends on the blocks an SM holds)."""
    if len(seen_variants) < 4:
        pytest.skip("runs after test_decode_attention_with_many_pairs_one_block_per_pair")
    assert {2, 3} <= set(seen_variants.values()), f"tile buffers seen: {sorted(seen_variants.items())}"


@pytest.mark.parametrize("n_seqs", [40, 64])
def test_fused_decode_attention_with_many_pairs(n_seqs):
    kernels.fused_decode_case(32, 8, 128, None, torch.float32, spread_lengths(n_seqs))
    assert ops().lib().thn_attention_decode_last_variant() % 10 == (2 if n_seqs == 64 else 0)
    try:
        ops().lib().thn_set_decode_stream(2, 3)
        kernels.fused_decode_case(32, 8, 128, None, torch.float32, spread_lengths(n_seqs))
        assert ops().lib().thn_attention_decode_last_variant() % 10 == 2
    finally:
        ops().lib().thn_set_decode_stream(1, 3)
    try:
        ops().lib().thn_set_decode_stream(0, 3)
        kernels.fused_decode_case(32, 8, 128, None, torch.float32, spread_lengths(n_seqs))
        assert ops().lib().thn_attention_decode_last_variant() % 10 == 0
    finally:
        ops().lib().thn_set_decode_stream(1, 3)


@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 64, None), (32, 8, 128, None), (6, 3, 64, 70), (3, 1, 128, 24),
                                               (16, 1, 64, None), (5, 5, 128, 200), (16, 1, 128, None), (32, 2, 128, 90)])
def test_streaming_decode_attention_at_other_sizes(streaming_always, n_q, n_kv, D, window):
    """The streaming kernel at the sizes and windows of the split kernel's test: both head
    sizes, groups of 1 to 16 heads, windows inside a page and across pages; and in its fused
    form against the two separate kernels, bit for bit."""
    lengths = [700, 64, 65, 1, 333, 128]
    got, want = kernels.attention_case("decode1", torch.bfloat16, n_q, n_kv, D, lengths, [1] * len(lengths), window)
    assert ops().lib().thn_attention_decode_last_variant() == 32
    kernels.close(got, want, torch.bfloat16, "streaming decode attention")


def test_streaming_decode_attention_finds_a_far_key_and_the_windows_edge(streaming_always, monkeypatch):
    monkeypatch.setenv("THN_DECODE_SPLITS", "1")
    kernels.test_attention_finds_a_far_key("decode", torch.bfloat16)
    assert ops().lib().thn_attention_decode_last_variant() == 32
    kernels.test_attention_window_edge("decode", torch.bfloat16)
    assert ops().lib().thn_attention_decode_last_variant() == 32


@pytest.mark.parametrize("n_q,n_kv,D,window", [(8, 2, 128, None), (6, 6, 64, None), (16, 1, 128, 100), (12, 2, 64, None)])
def test_streaming_fused_decode_attention_at_other_sizes(streaming_always, monkeypatch, n_q, n_kv, D, window):
    monkeypatch.setenv("THN_DECODE_SPLITS", "1")
    kernels.fused_decode_case(n_q, n_kv, D, window, torch.bfloat16, [129, 64, 1, 300, 77, 640])
    assert ops().lib().thn_attention_decode_last_variant() == 32


@pytest.mark.parametrize("fused", [False, True], ids=["plain", "fused"])
def test_streaming_decode_attention_gives_the_same_bits_every_time(fused):
    """The streaming kernel's tile buffers go round between the loader's copies (asynchronous
    proxy) and the warps' reads (generic proxy); handed back a moment too early, a buffer was
    once refilled under a read, in one launch out of four and only with two blocks on an SM.
    Two hundred launches on the same cache must all give the bits of the first, and those
    must be the bits of the kernel that takes one block per pair."""
    o = ops()
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    dtype, n_seqs, n_q, n_kv, D = torch.bfloat16, 48, 32, 8, 128
    lengths = spread_lengths(n_seqs)
    fix = kernels.PagedFixture(n_kv, D, lengths, dtype)
    old = [n - 1 for n in lengths]
    live = [i for i, n in enumerate(old) if n > 0]
    keep = fix.slots
    fix.slots = [keep[i] for i in live]
    rows, cu = fix.rows([old[i] for i in live])
    kernels.write_kv(fix, rows, kernels.rand((cu[-1], n_kv, D), dtype, 80), kernels.rand((cu[-1], n_kv, D), dtype, 81), n_q)
    fix.advance(rows, [old[i] for i in live])
    fix.slots = keep
    rows, cu = fix.rows([1] * n_seqs)
    err = o.new_error_word(DEV)
    scale = D ** -0.5
    if fused:
        rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": 1e4}), Runtime(dtype, torch.device(DEV), {}))
        rope.ensure(1024)
        qkv = kernels.rand((n_seqs, (n_q + 2 * n_kv) * D), dtype, 82, 2.0).to(DEV)
        gain = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(83))).to(DEV)

        def launch():
            return o.qkv_attention(qkv, gain, gain, 1e-6, rope.tables(), rows, fix.kv, n_q, scale, None, True, err)
    else:
        kernels.write_kv(fix, rows, kernels.rand((n_seqs, n_kv, D), dtype, 84), kernels.rand((n_seqs, n_kv, D), dtype, 85), n_q)
        q = kernels.rand((n_seqs, n_q * D), dtype, 86).to(DEV)

        def launch():
            return o.attention_decode_bf16(q, rows, fix.kv, n_q, scale, None, err, n_splits=1)
    o.lib().thn_set_decode_stream(2, 3)
    outs = [launch() for _ in range(200)]
    assert o.lib().thn_attention_decode_last_variant() == 32
    try:
        o.lib().thn_set_decode_stream(0, 3)
        one_block_per_pair = launch()
        assert o.lib().thn_attention_decode_last_variant() % 10 == 0
    finally:
        o.lib().thn_set_decode_stream(1, 3)
    assert int(err.item()) == 0
    differing = [i for i, out in enumerate(outs) if not torch.equal(out, outs[0])]
    assert not differing, f"launches {differing[:10]} of 200 differ from the first"
    worst = (outs[0].float() - one_block_per_pair.float()).abs().max().item()
    assert worst <= 2e-3, f"differs from the one-block-per-pair kernel by {worst:.3e}"


def test_many_long_sequences_go_to_the_streaming_kernel_by_the_hosts_hint():
    """16 sequences on 8 kv heads are fewer pairs than the GPU holds blocks, so by their number
    alone they would meet in clusters; told that they may hold a thousand keys and more, the
    launcher leaves the key ranges whole and streams them.  The result is the same either way."""
    o = ops()
    dtype, n_q, n_kv, D = torch.bfloat16, 32, 8, 128
    lengths = [1500, 1100, 40, 2000] * 4
    fix = kernels.PagedFixture(n_kv, D, lengths, dtype)
    rows, cu = fix.rows(lengths)
    kernels.write_kv(fix, rows, kernels.rand((cu[-1], n_kv, D), dtype, 90), kernels.rand((cu[-1], n_kv, D), dtype, 91), n_q)
    fix.advance(rows, lengths)
    fix.cache.seq_lens -= 1                                   # the step's token is the last one written
    rows = o.step_rows(torch.arange(len(lengths) + 1, dtype=torch.int32, device=DEV),
                       torch.tensor(fix.slots, dtype=torch.int32, device=DEV), fix.cache.seq_lens, len(lengths), 1)
    q = kernels.rand((len(lengths), n_q * D), dtype, 92).to(DEV)
    err = o.new_error_word(DEV)
    unhinted = o.attention_decode_bf16(q, rows, fix.kv, n_q, D ** -0.5, None, err)
    assert o.lib().thn_attention_decode_last_variant() % 10 == 1        # clusters
    rows.max_context, rows.lengths_differ = max(lengths), False       # (told so; the kernels believe the host)
    assert o.decode_splits(len(lengths), n_kv, DEV, D, context=rows.max_context, differ=False) == 1
    assert o.decode_splits(len(lengths), n_kv, DEV, D, context=rows.max_context, differ=True) > 1   # too few to pair up
    hinted = o.attention_decode_bf16(q, rows, fix.kv, n_q, D ** -0.5, None, err)
    assert o.lib().thn_attention_decode_last_variant() == 32            # streaming
    rows.max_context = 700                                                # short: clusters again
    o.attention_decode_bf16(q, rows, fix.kv, n_q, D ** -0.5, None, err)
    assert o.lib().thn_attention_decode_last_variant() % 10 == 1
    assert int(err.item()) == 0
    kernels.close(hinted, unhinted, dtype, "hinted against unhinted")
    assert (hinted.float() - unhinted.float()).abs().max().item() <= 2e-3


def test_decode_attention_few_pairs_meets_in_a_cluster():
    """The counterpart: few pairs, splits that meet in a cluster's shared memory."""
    lengths = [700, 64, 65, 1, 333, 128]
    got, want = kernels.attention_case("decode", torch.bfloat16, 32, 8, 128, lengths, [1] * 6, None)
    kernels.close(got, want, torch.bfloat16, "decode attention, few pairs")
    assert ops().lib().thn_attention_decode_last_variant() % 10 == 1


# ----------------------------------------------------------------------------- the head at its real width


def test_head_product_at_full_vocabulary():
    """8 rows against a 151,936 x 2,560 weight (the Qwen3-4B head): 1,187 tiles of 128 rows in
    balanced runs over the SMs, shared tiles summed by the last arriver, float32 out."""
    o = ops()
    m, n, k = 8, 151936, 2560
    g = torch.Generator(device=DEV).manual_seed(5)
    x = torch.randn((m, k), generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    err = o.new_error_word(DEV)
    before = o.calls_by_entry.get("thn_gemm_stream_bf16", 0)
    out = o.linear(x, w, out_dtype=torch.float32, err=err)
    assert o.calls_by_entry.get("thn_gemm_stream_bf16", 0) == before + 1, "the head went to the vendor library"
    assert int(err.item()) == 0, "a pipeline wait timed out"
    exact = torch.empty((m, n), dtype=torch.float64, device=DEV)
    for start in range(0, n, 16384):                       # in slices: float64 copies of the weight are large
        exact[:, start:start + 16384] = x.double() @ w[start:start + 16384].double().t()
    bound = 2e-6 * k ** 0.5 * max(1.0, exact.abs().max().item())      # the measure of test_gemm_stream
    worst = (out.double() - exact).abs().max().item()
    assert worst <= bound, f"error {worst:.3e} beyond {bound:.3e}"
    again = o.linear(x, w, out_dtype=torch.float32, err=err)
    assert torch.equal(out, again), "two runs differ: the order of the sum depends on timing"
    # ragged last tile (151,936 = 1,187 * 128 exactly; one row less leaves a tile of 127)
    short = o.linear(x, w[:-1].contiguous(), out_dtype=torch.float32, err=err)
    assert torch.equal(short, out[:, :-1])
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- generation at real sizes


def engine_at_real_sizes(folder, **kwargs):
    from thing_htn_2026_b200 import Engine
    return Engine(folder, dtype="bfloat16", **kwargs)


def test_captured_decode_program_gives_plain_logits(model_dir):  # noqa: F811
    """Generation's own single-token program, replayed as a CUDA graph: the fused decode
    attention at head size 128 with its cluster merge, the streaming tcgen05 products for o,
    down and the head, programmatic dependent launch between all of them.  The logits the
    graph leaves behind are compared with the plain implementation at every step; the tokens
    fed back are the engine's own greedy choices."""
    o = ops()
    from thing_htn_2026_b200.engine.generation import Request
    engine = engine_at_real_sizes(model_dir, max_tokens=1024, max_batch=4)
    backend = engine.backend
    prompts = [requests()[k][:n] for k, n in (("r0", 150), ("r1", 64), ("r2", 1))]
    n_new = 24
    stream_before = o.calls_by_entry.get("thn_gemm_stream_bf16", 0)
    fused_before = o.calls_by_entry.get("thn_attention_decode_fused_bf16", 0)
    with torch.inference_mode():
        slots = backend.open_batch([Request(p, n_new + 1, 0.0, 0, i) for i, p in enumerate(prompts)])
        emitted = [[t] for t in backend.fetch(backend.launch_prefill(slots, prompts))]
        step_logits = []
        for _ in range(n_new):
            tokens = backend.fetch(backend.launch_decode(slots))
            (key,) = [k for k in backend.graph_logits if k[0] == len(slots)]
            step_logits.append(backend.graph_logits[key].float().cpu().numpy().copy())
            for seq, t in zip(emitted, tokens):
                seq.append(t)
        backend.close_batch(slots)
    assert backend.graphs, "no graph was captured"
    # recorded into the graph once: per layer an o and a down product, and the head; the fused attention per layer
    layers = CONFIG["num_hidden_layers"]
    assert o.calls_by_entry.get("thn_gemm_stream_bf16", 0) - stream_before >= 2 * layers + 1
    assert o.calls_by_entry.get("thn_attention_decode_fused_bf16", 0) - fused_before >= layers
    for i, prompt in enumerate(prompts):
        full = prompt + emitted[i]
        got = np.stack([step[i] for step in step_logits])                 # logits after token len(prompt) + n
        want_places = slice(len(prompt), len(prompt) + n_new)
        exact = harness.plain_logits(model_dir, full, torch.float32)[want_places]
        rounded = harness.plain_logits(model_dir, full, torch.bfloat16)[want_places]
        noise = np.abs(harness.plain_logits(model_dir, full, torch.bfloat16)
                       - harness.plain_logits(model_dir, full, torch.float32)).max()
        assert np.abs(got - rounded).max() <= noise + 1e-3, f"sequence {i}: graph logits against plain bfloat16"
        assert np.abs(got - exact).max() <= 2 * noise + 1e-3, f"sequence {i}: graph logits against float32"
        for n in range(n_new):
            assert emitted[i][n + 1] == int(np.argmax(got[n])), "the token fed back is not the graph's own argmax"


def test_generate_at_real_sizes_graphs_on_and_off(model_dir):  # noqa: F811
    """Through the entry point, three unequal prompts, 40 greedy tokens, three steps in
    flight: every token is the plain argmax up to the measured bfloat16 margin, and eager
    steps choose the same tokens as the graphs."""
    import test_generate_gpu as gen
    prompts = [requests()[k][:n] for k, n in (("r0", 120), ("r1", 33), ("r2", 70))]
    tokens, steps = gen.collect(engine_at_real_sizes(model_dir, graphs=True, depth=3), prompts, 40)
    assert len(steps) == 40
    full = prompts[0] + tokens[0]
    noise = np.abs(harness.plain_logits(model_dir, full, torch.bfloat16)
                   - harness.plain_logits(model_dir, full, torch.float32)).max()
    for prompt, emitted in zip(prompts, tokens):
        logits = harness.plain_logits(model_dir, prompt + emitted, torch.bfloat16)
        for n, token in enumerate(emitted):
            row = logits[len(prompt) + n - 1]
            assert row[token] >= row.max() - (4 * noise + 1e-3), f"token {n}: {token} against plain argmax {row.argmax()}"
    eager, _ = gen.collect(engine_at_real_sizes(model_dir, graphs=False, depth=1), prompts, 40)
    assert eager == tokens


def test_generate_batch_64_at_real_sizes(model_dir, tmp_path):  # noqa: F811
    """64 sequences of unequal lengths: 512 (sequence, kv head) pairs in the decode attention,
    more rows than the streaming products take, until half of them end and the rest go on
    as a batch of 32.  Three sequences are held to the plain
    implementation; every sequence's tokens are checked against this library's replay of
    prompt + tokens (itself held to the plain implementation in test_real_sizes_gpu.py)."""
    import test_generate_gpu as gen
    g = torch.Generator().manual_seed(9)
    lens = [1 + int(x) for x in torch.randint(0, 90, (64,), generator=g)]
    prompts = [torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for n in lens]
    limits = [10 if i % 2 else 6 for i in range(64)]        # half end earlier: steps of 64 rows, then of 32
    engine = engine_at_real_sizes(model_dir, graphs=True, depth=3)
    tokens, steps = gen.collect(engine, prompts, limits)
    assert len(steps) == 10 and [len(t) for t in tokens] == limits
    assert {k[0] for k in engine.backend.graphs} == {64, 32}
    reqs = {f"s{i}": prompts[i] + tokens[i] for i in range(64)}
    replayed = harness.replay(model_dir, "bfloat16", harness.trace_whole(reqs), str(tmp_path))
    probe = reqs["s0"]
    noise = np.abs(harness.plain_logits(model_dir, probe, torch.bfloat16)
                   - harness.plain_logits(model_dir, probe, torch.float32)).max()
    for i in range(64):
        logits = replayed[f"s{i}"]
        for n, token in enumerate(tokens[i]):
            row = logits[len(prompts[i]) + n - 1]
            assert row[token] >= row.max() - (4 * noise + 1e-3), f"sequence {i} token {n}"
    harness.check_against_plain({k: replayed[k] for k in ("s0", "s1", "s2")}, {k: reqs[k] for k in ("s0", "s1", "s2")},
                                model_dir, "bfloat16", "batch 64")


def test_more_steps_in_flight_than_the_default_ring(tiny_models):
    """Twelve steps ahead of the host: the ring of pinned token buffers follows the depth, so
    no buffer is written again before the host has read it."""
    import test_generate_gpu as gen
    import tiny
    from thing_htn_2026_b200 import Engine
    prompts = [tiny.tokens("d", n, 900 + i) for i, n in enumerate([9, 30, 2])]
    deep, _ = gen.collect(Engine(tiny_models["d"], dtype="float32", depth=12), prompts, 40)
    shallow, _ = gen.collect(Engine(tiny_models["d"], dtype="float32", depth=1), prompts, 40)
    assert deep == shallow
    engine = Engine(tiny_models["d"], dtype="float32", depth=2)
    assert len(engine_backend_ring(engine, prompts)) == 4


def engine_backend_ring(engine, prompts):
    list(engine.generate(prompts, 2))
    return engine.backend._ring


def test_backend_refuses_to_overwrite_an_unfetched_step(tiny_models):
    from thing_htn_2026_b200 import Engine
    from thing_htn_2026_b200.engine.generation import Request
    engine = Engine(tiny_models["a"], dtype="float32", max_tokens=256, depth=1)       # a ring of three
    backend = engine.backend
    with torch.inference_mode():
        slots = backend.open_batch([Request([1, 2, 3], 20)])
        handles = [backend.launch_prefill(slots, [[1, 2, 3]])] + [backend.launch_decode(slots) for _ in range(2)]
        with pytest.raises(RuntimeError, match="steps are in flight"):
            backend.launch_decode(slots)
        for h in handles:
            backend.fetch(h)
        backend.fetch(backend.launch_decode(slots))
        backend.close_batch(slots)


# ----------------------------------------------------------------------------- the device error word


def error_case(kernel, break_what):
    """A step whose block table lacks a page the step reads, or whose rotary table is shorter
    than a position; returns the error word's bits.  The kernels skip the access."""
    o = ops()
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    dtype = torch.float32 if kernel == "generic32" else torch.bfloat16
    n_q, n_kv, D = 8, 2, 128
    lengths = [300, 70]
    counts = [1, 1] if kernel in ("decode", "fused", "generic32") else [150, 70]
    fix = kernels.PagedFixture(n_kv, D, lengths, dtype)
    old = [n - c for n, c in zip(lengths, counts)]
    live = [i for i, n in enumerate(old) if n > 0]
    keep = fix.slots
    if live:
        fix.slots = [keep[i] for i in live]
        rows, _ = fix.rows([old[i] for i in live])
        fix.advance(rows, [old[i] for i in live])
        fix.slots = keep
    rows, cu = fix.rows(counts)
    rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": 1e4}), Runtime(dtype, torch.device(DEV), {}))
    rope.ensure(512)
    tables = rope.tables()
    if break_what == "page":
        fix.kv.block_table[fix.slots[0], 1] = -1              # positions 64..127 of the first sequence
    else:
        tables = o.RotaryTables(tables.cos[:200].contiguous(), tables.sin[:200].contiguous(), tables.rotary_dim)
    err = o.new_error_word(DEV)
    scale = D ** -0.5
    q = kernels.rand((cu[-1], n_q * D), dtype, 1).to(DEV)
    qkv = kernels.rand((cu[-1], (n_q + 2 * n_kv) * D), dtype, 2).to(DEV)
    gain = torch.ones(D, dtype=torch.float32, device=DEV)
    if kernel in ("generic", "generic32"):
        o.attention_generic(q, rows, fix.kv, n_q, scale, None, err)
    elif kernel == "prefill":
        o.attention_prefill_bf16(q, rows, rows.tiles, fix.kv, n_q, scale, None, err)
    elif kernel == "tcgen05":
        o.attention_prefill_tcgen05(q, rows, rows.tiles, fix.kv, n_q, scale, None, err)
    elif kernel == "decode":
        o.attention_decode_bf16(q, rows, fix.kv, n_q, scale, None, err)
    elif kernel == "fused":
        o.qkv_attention(qkv, gain, gain, 1e-6, tables, rows, fix.kv, n_q, scale, None, True, err)
    elif kernel == "rope":
        o.qk_norm_rope_cache(qkv, gain, gain, 1e-6, tables, rows, fix.kv, n_q, True, err)
    torch.cuda.synchronize()
    bits = int(err.item())
    with pytest.raises(o.KernelError, match="device reported"):
        o.raise_on_device_error(err, "test")
    assert int(err.item()) == 0, "raising clears the word"
    return bits


@pytest.mark.parametrize("kernel", ["generic32", "generic", "prefill", "decode", "fused", "tcgen05"])
def test_unmapped_page_sets_its_bit(kernel):
    o = ops()
    bits = error_case(kernel, "page")
    assert bits & o.ERR_PAGE_UNMAPPED, f"error word {bits}"
    assert bits == o.ERR_PAGE_UNMAPPED


def test_a_wait_that_runs_out_sets_its_bit_and_the_kernel_returns():
    """The tcgen05 prompt attention with its loader told (by a switch that exists for this
    test) to bring no key or value page: the waits for them are bounded by a clock, run out
    after 20 ms, set their bit, and every block leaves through its common exit.  The next
    launch, with the switch off, is right again."""
    o = ops()
    assert o.lib().thn_attention_tcgen05_test_skip_loads(1) == 0
    try:
        fix = kernels.PagedFixture(2, 128, [70], torch.bfloat16)
        rows, cu = fix.rows([70])
        q = kernels.rand((70, 4 * 128), torch.bfloat16, 1).to(DEV)
        err = o.new_error_word(DEV)
        o.attention_prefill_tcgen05(q, rows, rows.tiles, fix.kv, 4, 128 ** -0.5, None, err)
        torch.cuda.synchronize()
        assert int(err.item()) == o.ERR_WAIT_TIMEOUT
    finally:
        assert o.lib().thn_attention_tcgen05_test_skip_loads(0) == 0
    got, want = kernels.attention_case("tcgen05", torch.bfloat16, 4, 2, 128, [70, 131], [70, 131], None)
    kernels.close(got, want, torch.bfloat16, "tcgen05 attention after a timed-out launch")


@pytest.mark.parametrize("kernel", ["rope", "fused"])
def test_position_beyond_the_rotary_table_sets_its_bit(kernel):
    o = ops()
    assert error_case(kernel, "position") == o.ERR_POSITION_RANGE
