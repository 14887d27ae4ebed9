"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's
tiny configurations: widths and vocabularies that are no power of two, head sizes in steps
of 16, odd head counts and groups; in float32 and in bfloat16."""

import numpy as np
import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from thing_htn_2026_b200 import ops as module
    return module


def close(got, want, dtype, what, scale=1.0):
    """float32: sums in another order.  bfloat16: the reference's own rule for a kernel
    against its twin, |a - b| <= 1e-2 + |b| / 64 (engine/engine.py:425-429)."""
    got, want = got.float().cpu(), want.float().cpu()
    if dtype == torch.float32:
        err = (got - want).abs().max().item()
        assert err <= 2e-5 * scale * max(1.0, want.abs().max().item()), f"{what}: float32 differs by {err:.3e}"
    else:
        bad = (got - want).abs() > 1e-2 + want.abs() / 64
        assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} bfloat16 values out of tolerance"


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ----------------------------------------------------------------------------- elementwise


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 128), (6, 2560), (37, 1000), (3, 96), (5, 77)])
def test_rmsnorm_and_add(dtype, rows, width):
    x, d = rand((rows, width), dtype, 1, 3.0), rand((rows, width), dtype, 2)
    for gain_dtype in ([dtype] if dtype == torch.float32 else [torch.bfloat16, torch.float32]):
        w = (1 + 0.5 * torch.randn(width, generator=torch.Generator().manual_seed(3))).to(gain_dtype)
        y = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5)
        close(y, plain.rms_norm(x, w, 1e-5, dtype), dtype, "rmsnorm")
        h = x.clone().to(DEV)
        y = ops().add_rmsnorm(h, d.to(DEV), w.to(DEV), 1e-6)
        h_want = plain.add_residual(x, d, dtype)
        assert torch.equal(h.cpu(), h_want), "residual sum is rounded once and must be exact"
        close(y, plain.rms_norm(h_want, w, 1e-6, dtype), dtype, "add_rmsnorm")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(1, 9728), (7, 100), (64, 333)])
def test_swiglu(dtype, rows, inter):
    gu = rand((rows, 2 * inter), dtype, 4, 4.0)
    out = ops().swiglu(gu.to(DEV))
    close(out, plain.swiglu(gu[:, :inter], gu[:, inter:], dtype), dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_rows_and_range_check(dtype):
    table = rand((301, 72), dtype, 5)
    index = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32)
    err = ops().new_error_word(DEV)
    out = ops().gather_rows(table.to(DEV), index.to(DEV), err)
    assert torch.equal(out.cpu(), table[index.long()])
    assert int(err.item()) == 0
    ops().gather_rows(table.to(DEV), torch.tensor([301], dtype=torch.int32, device=DEV), err)
    with pytest.raises(ops().KernelError, match="outside the vocabulary"):
        ops().raise_on_device_error(err, "test")


@pytest.mark.parametrize("m,n,k", [(1, 100, 64), (5, 77, 130), (64, 64, 16), (130, 200, 333)])
def test_gemm_f32_is_true_float32(m, n, k):
    a, w = rand((m, k), torch.float32, 6), rand((n, k), torch.float32, 7)
    out = ops().linear(a.to(DEV), w.to(DEV)).cpu()
    exact = (a.double() @ w.double().t())
    err = (out.double() - exact).abs().max().item()
    assert err <= 4e-7 * k ** 0.5 * exact.abs().max().item() + 1e-6, f"error {err:.3e} is not float32-like"
    # a row's result does not depend on the other rows of the call
    alone = ops().linear(a[:1].contiguous().to(DEV), w.to(DEV)).cpu()
    assert torch.equal(alone[0], out[0])


def test_rope_table_matches_formula():
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    for head_dim, theta in [(16, 1e4), (48, 5e5), (128, 5e6)]:
        rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": head_dim, "theta": theta}),
                                              Runtime(torch.float32, torch.device(DEV), {}))
        rope.ensure(3000)
        cos, sin = plain.rope_cos_sin(torch.arange(3000), head_dim, theta, torch.float32)
        t = rope.tables()
        assert (t.cos[:3000].cpu() - cos[:, :head_dim // 2]).abs().max() <= 2e-6
        assert (t.sin[:3000].cpu() - sin[:, :head_dim // 2]).abs().max() <= 2e-6


@pytest.mark.parametrize("m", [1, 8, 9, 16, 17, 40, 64])
@pytest.mark.parametrize("n,k", [(100, 64), (2560, 4096), (6144, 2560), (77, 648), (2560, 9728), (300, 72)])
def test_gemm_stream(m, n, k):
    """The TMA / tcgen05 weight-streaming product against a float64 product, with the work cut
    for the whole GPU and for odd numbers of blocks (tiles shared by 1 to many blocks, runs
    that start and end inside tiles, N and K that leave ragged tiles) and with each tile cut
    along K inside a thread-block cluster; the result does not depend on the run at all, and
    a row does not depend on the rows beside it."""
    o = ops()
    x, w = rand((m, k), torch.bfloat16, 60), rand((n, k), torch.bfloat16, 61, 0.05)
    exact = x.double() @ w.double().t()
    bound = 2e-6 * k ** 0.5 * max(1.0, exact.abs().max().item())
    err = o.new_error_word(DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    for n_blocks in [0, 1, 7, 1000, -2, -6]:           # negative: a thread-block cluster of that size per tile
        out32 = o.linear_stream(xd, wd, torch.float32, err=err, n_blocks=n_blocks)
        assert int(err.item()) == 0, "a pipeline wait timed out"
        worst = (out32.double().cpu() - exact).abs().max().item()
        assert worst <= bound, f"n_blocks {n_blocks}: error {worst:.3e}"
        out16 = o.linear_stream(xd, wd, err=err, n_blocks=n_blocks)
        assert torch.equal(out16, out32.to(torch.bfloat16)), "bfloat16 output is the float32 sum rounded once"
        again = o.linear_stream(xd, wd, torch.float32, err=err, n_blocks=n_blocks)
        assert torch.equal(again, out32), "two runs differ: the order of the sum depends on timing"
    whole = o.linear_stream(xd, wd, torch.float32, err=err)
    alone = o.linear_stream(xd[m - 1:].contiguous(), wd, torch.float32, err=err)
    assert torch.equal(whole[m - 1:], alone), "a row depends on its batch mates"
    assert int(err.item()) == 0


@pytest.mark.parametrize("m,inter,k", [(1, 128, 64), (8, 9728, 2560), (13, 200, 136), (33, 384, 200), (64, 1000, 512)])
def test_gemm_stream_fused_swiglu(m, inter, k):
    """Gate/up product and SwiGLU in one weight-streaming kernel against the two plain steps;
    the measure is the one of the many-row fused kernel."""
    o = ops()
    x, w = rand((m, k), torch.bfloat16, 62), rand((2 * inter, k), torch.bfloat16, 63, 0.05)
    err = o.new_error_word(DEV)
    gu = x.float() @ w.float().t()
    want = plain.swiglu(gu[:, :inter].to(torch.bfloat16), gu[:, inter:].to(torch.bfloat16), torch.bfloat16).float()
    exact = plain.swiglu(gu[:, :inter], gu[:, inter:], torch.float32)
    noise = (want - exact).abs()
    step = torch.exp2(torch.floor(torch.log2(want.abs().clamp_min(1e-30))) - 7)
    for n_blocks in [0, 5]:
        out = o.linear_stream(x.to(DEV), w.to(DEV), err=err, swiglu=True, n_blocks=n_blocks).float().cpu()
        assert int(err.item()) == 0, "a pipeline wait timed out"
        err_abs = (out - want).abs()
        assert (err_abs - step).max() <= noise.max(), f"{(err_abs - step).max():.3e} beyond a rounding step"
        assert err_abs.pow(2).mean().sqrt() <= noise.pow(2).mean().sqrt() + 1e-12


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (100, 200, 72), (300, 1000, 136), (2048, 2560, 4096), (513, 6144, 2560),
                                   (64, 2560, 9728)])
def test_gemm_tcgen05(m, n, k):
    """The tcgen05 / TMEM / TMA product against a float64 product: whole tiles, ragged edges in
    every dimension, several tiles per block, deep and shallow reductions."""
    o = ops()
    x, w = rand((m, k), torch.bfloat16, 50), rand((n, k), torch.bfloat16, 51, 0.05)
    err = o.new_error_word(DEV)
    out = o.linear_tcgen05(x.to(DEV), w.to(DEV), err)
    assert int(err.item()) == 0, "a pipeline wait timed out"
    exact = x.double() @ w.double().t()
    close(out, exact.to(torch.bfloat16), torch.bfloat16, "tcgen05 product")
    again = o.linear_tcgen05(x.to(DEV), w.to(DEV), err)
    assert torch.equal(out, again)


@pytest.mark.parametrize("m,inter,k", [(128, 128, 64), (300, 384, 200), (2048, 9728, 2560)])
def test_gemm_tcgen05_fused_swiglu(m, inter, k):
    """Gate/up product and SwiGLU in one kernel against the two plain steps.  g and u are
    rounded to bfloat16 before the activation, as the separate product stores them; a sum in
    another order flips such a rounding now and then, and the flip is carried through the
    activation and the product, so the measure is bfloat16's own noise on this input (plain
    bfloat16 against plain float32) plus one rounding step of the result."""
    o = ops()
    x, w = rand((m, k), torch.bfloat16, 52), rand((2 * inter, k), torch.bfloat16, 53, 0.05)
    err = o.new_error_word(DEV)
    out = o.linear_tcgen05(x.to(DEV), w.to(DEV), err, swiglu=True).float().cpu()
    assert int(err.item()) == 0, "a pipeline wait timed out"
    gu = x.float() @ w.float().t()
    want = plain.swiglu(gu[:, :inter].to(torch.bfloat16), gu[:, inter:].to(torch.bfloat16), torch.bfloat16).float()
    exact = plain.swiglu(gu[:, :inter], gu[:, inter:], torch.float32)
    noise = (want - exact).abs()
    step = torch.exp2(torch.floor(torch.log2(want.abs().clamp_min(1e-30))) - 7)
    err_abs = (out - want).abs()
    assert (err_abs - step).max() <= noise.max(), f"{(err_abs - step).max():.3e} beyond a rounding step"
    assert err_abs.pow(2).mean().sqrt() <= noise.pow(2).mean().sqrt()


# ----------------------------------------------------------------------------- cache helpers


class PagedFixture:
    """A cache with one entry, sequences of given lengths on scrambled pages."""

    def __init__(self, n_kv, head_dim, lengths, dtype, window=None, seed=0):
        from thing_htn_2026_b200.cache import KVSpec, SequenceCache
        self.lengths = lengths
        total = sum(-(-n // 64) * 64 for n in lengths) + 5 * 64
        self.cache = SequenceCache([KVSpec(n_kv, head_dim, window)], max_tokens=total, dtype=dtype, device=DEV,
                                   max_slots=len(lengths) + 3)
        # take and give back a few pages and slots so that ids are not 0, 1, 2, ...
        junk = self.cache.open(2)
        self.cache.prepare(junk, [130, 70])
        self.slots = self.cache.open(len(lengths))
        self.cache.close(junk[:1])
        self.kv = self.cache.kv_view(0)
        self.dtype = dtype

    def rows(self, counts):
        """Step rows for ``counts[i]`` new tokens of sequence i (pages get mapped)."""
        o = ops()
        self.cache.prepare(self.slots, counts)
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
        slots_dev = torch.tensor(self.slots, dtype=torch.int32, device=DEV)
        rows = o.step_rows(cu_dev, slots_dev, self.cache.seq_lens, cu[-1], max(counts))
        rows.tiles = None
        if max(counts) > 1:
            size = o.ROW_TILE()
            held = [self.cache.length(slot) for slot in self.slots]
            r0, rn = o.row_tiles_of(counts, held, size)
            rows.tiles = o.RowTiles(torch.tensor(r0, dtype=torch.int32, device=DEV),
                                    torch.tensor(rn, dtype=torch.int32, device=DEV), len(r0), size)
        return rows, cu

    def advance(self, rows, counts):
        ops().advance(self.cache.seq_lens, rows.slots, rows.cu_seqlens)
        self.cache.commit(self.slots, counts)


def write_kv(fix, rows, k, v, n_q):
    """Puts k, v [rows, n_kv, D] into the cache through the library's own kernel (no norm,
    no rotation) and returns nothing."""
    o = ops()
    n_kv, D = fix.kv.n_kv, fix.kv.head_dim
    qkv = torch.cat([torch.zeros(k.shape[0], n_q * D, dtype=k.dtype), k.reshape(k.shape[0], -1),
                     v.reshape(v.shape[0], -1)], dim=1).to(DEV)
    err = o.new_error_word(DEV)
    o.qk_norm_rope_cache(qkv, None, None, 1.0, None, rows, fix.kv, n_q, True, err)
    assert int(err.item()) == 0


def attention_case(kernel, dtype, n_q, n_kv, D, lengths, new_counts, window, seed=0, peak=None):
    """Sequences with ``lengths[i]`` tokens in all, the last ``new_counts[i]`` of which are
    this step's rows.  Returns (got, want) for the step's rows."""
    o = ops()
    fix = PagedFixture(n_kv, D, lengths, dtype, window)
    total = sum(lengths)
    q_all = [rand((n, n_q, D), dtype, seed + 10 * i + 1) for i, n in enumerate(lengths)]
    k_all = [rand((n, n_kv, D), dtype, seed + 10 * i + 2) for i, n in enumerate(lengths)]
    v_all = [rand((n, n_kv, D), dtype, seed + 10 * i + 3) for i, n in enumerate(lengths)]
    if peak is not None:
        peak(q_all, k_all, v_all)
    # first step: the old tokens (keys and values only)
    old = [n - c for n, c in zip(lengths, new_counts)]
    if max(old) > 0:
        live = [i for i, n in enumerate(old) if n > 0]
        fix_slots = fix.slots
        fix.slots = [fix_slots[i] for i in live]
        rows, _ = fix.rows([old[i] for i in live])
        write_kv(fix, rows, torch.cat([k_all[i][:old[i]] for i in live]), torch.cat([v_all[i][:old[i]] for i in live]),
                 n_q)
        fix.advance(rows, [old[i] for i in live])
        fix.slots = fix_slots
    rows, cu = fix.rows(new_counts)
    write_kv(fix, rows, torch.cat([k[-c:] for k, c in zip(k_all, new_counts)]),
             torch.cat([v[-c:] for v, c in zip(v_all, new_counts)]), n_q)
    q = torch.cat([x[-c:] for x, c in zip(q_all, new_counts)]).reshape(cu[-1], n_q * D).to(DEV)
    err = o.new_error_word(DEV)
    scale = D ** -0.5
    if kernel == "generic":
        got = o.attention_generic(q, rows, fix.kv, n_q, scale, window, err)
    elif kernel == "prefill":
        got = o.attention_prefill_bf16(q, rows, rows.tiles, fix.kv, n_q, scale, window, err)
    elif kernel == "tcgen05":
        got = o.attention_prefill_tcgen05(q, rows, rows.tiles, fix.kv, n_q, scale, window, err)
    elif kernel == "decode_long":
        rows.max_context = max(lengths)           # what the engine knows on the host
        got = o.attention_decode_bf16(q, rows, fix.kv, n_q, scale, window, err)
    elif kernel.startswith("decode"):
        got = o.attention_decode_bf16(q, rows, fix.kv, n_q, scale, window, err,
                                      n_splits=int(kernel[6:]) if len(kernel) > 6 else None)
    assert int(err.item()) == 0, f"device error word {int(err.item())}"
    want = torch.cat([plain.attention(qs, ks, vs, scale, window, dtype)[-c:]
                      for qs, ks, vs, c in zip(q_all, k_all, v_all, new_counts)])
    return got.cpu(), want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 16, None), (6, 3, 48, 20), (8, 1, 32, None), (5, 5, 80, 70),
                                               (4, 2, 128, None), (2, 1, 256, 100)])
def test_attention_generic(dtype, n_q, n_kv, D, window):
    got, want = attention_case("generic", dtype, n_q, n_kv, D, [70, 5, 131], [70, 5, 131], window)
    close(got, want, dtype, "generic attention, whole prompts", scale=4)
    got, want = attention_case("generic", dtype, n_q, n_kv, D, [200, 64, 65, 1], [1, 1, 1, 1], window)
    close(got, want, dtype, "generic attention, single tokens", scale=4)
    got, want = attention_case("generic", dtype, n_q, n_kv, D, [150, 90], [30, 64], window)
    close(got, want, dtype, "generic attention, continued prompts", scale=4)


@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 64, None), (8, 2, 128, None), (6, 3, 64, 70), (3, 1, 128, 24),
                                               (16, 1, 64, None), (5, 5, 128, 200)])
def test_attention_prefill_tensor_cores(n_q, n_kv, D, window):
    dtype = torch.bfloat16
    got, want = attention_case("prefill", dtype, n_q, n_kv, D, [70, 5, 131, 64, 1, 257], [70, 5, 131, 64, 1, 257], window)
    close(got, want, dtype, "prefill attention, whole prompts")
    got, want = attention_case("prefill", dtype, n_q, n_kv, D, [300, 90, 129], [170, 64, 1], window)
    close(got, want, dtype, "prefill attention, continued prompts")


@pytest.mark.parametrize("splits", ["", "1", "3", "8", "12"])
@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 32, None), (6, 3, 48, 70), (8, 2, 80, None), (16, 1, 96, None),
                                               (5, 5, 112, 200), (32, 2, 96, 90)])
def test_attention_tensor_cores_at_other_head_sizes(n_q, n_kv, D, window, splits):
    """Head sizes in steps of 16 between 32 and 128 other than 64 and 128: the same prompt and
    single-token kernels with two tile buffers, splits meeting in a cluster (3, 8) or through
    scratch memory (12), against the plain implementation."""
    dtype = torch.bfloat16
    assert ops().lib().thn_attention_mma_supported(D, 64, n_q, n_kv) == 1
    assert ops().lib().thn_attention_fused_supported(D, 64, n_q, n_kv) == 0
    lengths = [700, 64, 65, 1, 333, 128]
    got, want = attention_case("decode" + splits, dtype, n_q, n_kv, D, lengths, [1] * len(lengths), window)
    close(got, want, dtype, f"decode attention, head size {D}, splits {splits or 'auto'}")
    if splits == "":
        got, want = attention_case("prefill", dtype, n_q, n_kv, D, [70, 5, 131, 64, 1, 257], [70, 5, 131, 64, 1, 257], window)
        close(got, want, dtype, f"prefill attention, head size {D}, whole prompts")
        got, want = attention_case("prefill", dtype, n_q, n_kv, D, [300, 90, 129], [170, 64, 1], window)
        close(got, want, dtype, f"prefill attention, head size {D}, continued prompts")


def test_attention_head_sizes_the_tensor_core_kernels_refuse():
    o = ops()
    for D in (16, 24, 40, 136, 144, 256):
        assert o.lib().thn_attention_mma_supported(D, 64, 4, 2) == 0, D
    for D in (32, 48, 64, 80, 96, 112, 128):
        assert o.lib().thn_attention_mma_supported(D, 64, 4, 2) == 1, D
        assert o.lib().thn_attention_fused_supported(D, 64, 4, 2) == (1 if D in (64, 128) else 0), D
    assert o.lib().thn_attention_mma_supported(64, 64, 34, 2) == 0      # 17 query heads per kv head
    assert o.lib().thn_attention_mma_supported(64, 32, 4, 2) == 0       # pages of 32 tokens


@pytest.mark.parametrize("n_q,n_kv,window", [(2, 1, None), (8, 2, None), (6, 3, 70), (3, 1, 24), (5, 5, 200)])
def test_attention_prefill_tcgen05(n_q, n_kv, window):
    """The tcgen05 prompt kernel: whole prompts (one row to several tiles) and continued ones."""
    dtype, D = torch.bfloat16, 128
    got, want = attention_case("tcgen05", dtype, n_q, n_kv, D, [70, 5, 131, 64, 1, 257], [70, 5, 131, 64, 1, 257], window)
    close(got, want, dtype, "tcgen05 attention, whole prompts")
    got, want = attention_case("tcgen05", dtype, n_q, n_kv, D, [300, 90, 129, 500], [170, 64, 1, 300], window)
    close(got, want, dtype, "tcgen05 attention, continued prompts")


@pytest.mark.parametrize("splits", ["", "1", "3", "8", "12", "32"])
@pytest.mark.parametrize("n_q,n_kv,D,window", [(4, 2, 64, None), (32, 8, 128, None), (6, 3, 64, 70), (3, 1, 128, 24),
                                               (16, 1, 64, None), (5, 5, 128, 200), (16, 1, 128, None), (32, 2, 128, 90)])
def test_attention_decode_tensor_cores(n_q, n_kv, D, window, splits):
    """One block per sequence (1), splits that meet in a thread-block cluster's shared memory
    (3, 8) and splits that meet in global memory (12, 32: more than a cluster holds)."""
    dtype = torch.bfloat16
    lengths = [700, 64, 65, 1, 333, 128]
    got, want = attention_case("decode" + splits, dtype, n_q, n_kv, D, lengths, [1] * len(lengths), window)
    close(got, want, dtype, f"decode attention, splits {splits or 'auto'}")


@pytest.mark.parametrize("kernel,dtype", [("generic", torch.float32), ("generic", torch.bfloat16),
                                          ("prefill", torch.bfloat16), ("decode", torch.bfloat16),
                                          ("decode4", torch.bfloat16)])
def test_attention_finds_a_far_key(kernel, dtype):
    """One key among hundreds, far back, is made to dominate one query head: the output of
    that head must be that key's value row.  Random weights alone would average any
    mistake about far keys away."""
    n_q, n_kv, D = 4, 2, 64
    target = 37

    def peak(q_all, k_all, v_all):
        direction = torch.zeros(D)
        direction[5] = 1.0
        q_all[0][-1, 2] = (direction * 40).to(dtype)        # head 2 -> kv head 1
        k_all[0][target, 1] = (direction * 40).to(dtype)

    lengths = [600, 100]
    counts = [1, 1] if kernel.startswith("decode") else lengths
    holder = {}

    def keep(q_all, k_all, v_all):
        peak(q_all, k_all, v_all)
        holder["v"] = v_all[0][target, 1].float()

    got, want = attention_case(kernel, dtype, n_q, n_kv, D, lengths, counts, None, peak=keep)
    row = (0 if kernel.startswith("decode") else lengths[0] - 1)
    head = got[row].reshape(n_q, D)[2].float()
    assert (head - holder["v"]).abs().max() < 2e-2, "the far key did not win"
    close(got, want, dtype, "far key", scale=4)


def test_attention_decode_long_context_finds_a_far_key():
    """A step that is known to hold many keys divides each key range among more blocks than a
    cluster has.  One key thousands of places back dominates a head of the long sequence; a
    short sequence shares the step, and most of its splits are empty."""
    o = ops()
    dtype = torch.bfloat16
    n_q, n_kv, D = 4, 2, 128
    lengths = [o.LONG_CONTEXT + 150, 70]
    target = 4321
    assert o.decode_splits(len(lengths), n_kv, DEV, D, context=max(lengths)) > o.lib().thn_attention_decode_cluster_splits()
    assert o.decode_splits(len(lengths), n_kv, DEV, D, context=o.LONG_CONTEXT - 1) == o.decode_splits(len(lengths), n_kv, DEV, D)
    holder = {}

    def peak(q_all, k_all, v_all):
        direction = torch.zeros(D)
        direction[9] = 1.0
        q_all[0][-1, 3] = (direction * 40).to(dtype)        # head 3 -> kv head 1
        k_all[0][target, 1] = (direction * 40).to(dtype)
        holder["v"] = v_all[0][target, 1].float()

    got, want = attention_case("decode_long", dtype, n_q, n_kv, D, lengths, [1, 1], None, peak=peak)
    head = got[0].reshape(n_q, D)[3].float()
    assert (head - holder["v"]).abs().max() < 2e-2, "the far key did not win"
    close(got, want, dtype, "decode attention, long context", scale=4)


@pytest.mark.parametrize("kernel,dtype", [("generic", torch.float32), ("prefill", torch.bfloat16),
                                          ("decode", torch.bfloat16), ("decode3", torch.bfloat16)])
def test_attention_window_edge(kernel, dtype):
    """The last key inside the window and the first key outside it are both made to stand
    out: the inner one must win and the outer one must not be seen at all."""
    n_q, n_kv, D, window = 2, 1, 64, 70
    length = 200
    inner, outer = length - window, length - window - 1     # positions p - W + 1 and p - W for p = length - 1
    holder = {}

    def peak(q_all, k_all, v_all):
        direction = torch.zeros(D)
        direction[9] = 1.0
        q_all[0][-1, 0] = (direction * 30).to(dtype)
        k_all[0][inner, 0] = (direction * 30).to(dtype)
        k_all[0][outer, 0] = (direction * 60).to(dtype)      # would win by far if it were visible
        holder["inner"] = v_all[0][inner, 0].float()

    counts = [1] if kernel.startswith("decode") else [length]
    got, want = attention_case(kernel, dtype, n_q, n_kv, D, [length], counts, window, peak=peak)
    head = got[-1].reshape(n_q, D)[0].float()
    assert (head - holder["inner"]).abs().max() < 2e-2, "the window's edge is off by one"
    close(got, want, dtype, "window edge", scale=4)


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n_q,n_kv,D", [(5, 1, 64), (8, 2, 128), (3, 1, 256)])
def test_qk_norm_rope_cache_same_bits_for_long_and_short_steps(n_q, n_kv, D, gain_dtype):
    """Steps of many rows go through another kernel (16-byte accesses, paired bfloat16
    products) than steps of few rows; a token's q and its cache entry must not depend on
    which one it met: 200 rows in one step against the same rows in steps of 50."""
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    o = ops()
    dtype = torch.bfloat16
    rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": 4321.0}),
                                          Runtime(dtype, torch.device(DEV), {}))
    rope.ensure(256)
    qkv = rand((200, (n_q + 2 * n_kv) * D), dtype, 80, 2.0).to(DEV)
    qg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(81))).to(gain_dtype).to(DEV)
    kg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(82))).to(gain_dtype).to(DEV)
    err = o.new_error_word(DEV)
    results = []
    for chunk in (200, 50):
        fix = PagedFixture(n_kv, D, [200], dtype)
        parts = []
        for start in range(0, 200, chunk):
            rows, _ = fix.rows([chunk])
            parts.append(o.qk_norm_rope_cache(qkv[start:start + chunk].contiguous(), qg, kg, 1e-6, rope.tables(), rows,
                                              fix.kv, n_q, True, err))
            fix.advance(rows, [chunk])
        results.append((torch.cat(parts), fix.kv.storage.clone(), fix.kv.block_table.clone()))
    assert int(err.item()) == 0
    (q_long, cache_long, table_long), (q_short, cache_short, table_short) = results
    assert torch.equal(table_long, table_short)
    assert torch.equal(q_long, q_short), "q depends on the length of the step"
    assert torch.equal(cache_long, cache_short), "the cache depends on the length of the step"


# ----------------------------------------------------------------------------- fused single-token step


@pytest.mark.parametrize("gain_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n_q,n_kv,D,window", [(8, 2, 128, None), (6, 6, 64, None), (16, 1, 128, 100), (32, 8, 128, None),
                                               (12, 2, 64, None)])
def test_qkv_attention_fused_decode_equals_two_kernels(n_q, n_kv, D, window, gain_dtype):
    """A single-token step through the one fused kernel (q/k norm, rotation, cache write,
    attention) gives, bit for bit, the output and the cache of the two separate kernels.
    The lengths put the new token at a page's first row, at its last row and in the middle,
    and make one sequence one token long."""
    fused_decode_case(n_q, n_kv, D, window, gain_dtype, [129, 64, 1, 300, 77, 640])


def fused_decode_case(n_q, n_kv, D, window, gain_dtype, lengths):
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    o = ops()
    dtype = torch.bfloat16
    old = [n - 1 for n in lengths]
    fix = PagedFixture(n_kv, D, lengths, dtype, window)
    # the tokens before this step
    keep = fix.slots
    fix.slots = [s for s, n in zip(keep, old) if n]
    rows, cu = fix.rows([n for n in old if n])
    k = rand((cu[-1], n_kv, D), dtype, 70)
    v = rand((cu[-1], n_kv, D), dtype, 71)
    write_kv(fix, rows, k, v, n_q)
    fix.advance(rows, [n for n in old if n])
    fix.slots = keep

    rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": 54321.0}),
                                          Runtime(dtype, torch.device(DEV), {}))
    rope.ensure(1024)
    rows, cu = fix.rows([1] * len(lengths))
    qkv = rand((len(lengths), (n_q + 2 * n_kv) * D), dtype, 72, 2.0).to(DEV)
    qg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(73))).to(gain_dtype).to(DEV)
    kg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(74))).to(gain_dtype).to(DEV)
    err = o.new_error_word(DEV)
    before = fix.kv.storage.clone()
    scale = D ** -0.5

    q = o.qk_norm_rope_cache(qkv, qg, kg, 1e-6, rope.tables(), rows, fix.kv, n_q, True, err)
    want = o.attention(q, rows, fix.kv, n_q, scale, window, err)
    cache_want = fix.kv.storage.clone()
    assert not torch.equal(cache_want, before)

    fix.kv.storage.copy_(before)
    got = o.qkv_attention(qkv, qg, kg, 1e-6, rope.tables(), rows, fix.kv, n_q, scale, window, True, err)
    assert int(err.item()) == 0
    assert torch.equal(fix.kv.storage, cache_want), "the fused kernel leaves another cache"
    assert torch.equal(got, want), "the fused kernel gives another output"

    # a layer that reads another layer's cache: the token is there already, nothing is written
    got = o.qkv_attention(qkv, qg, kg, 1e-6, rope.tables(), rows, fix.kv, n_q, scale, window, False, err)
    assert torch.equal(got, want) and torch.equal(fix.kv.storage, cache_want)
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------- q/k norm, rotation, cache write


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lengths,counts", [([90, 7, 64], [25, 7, 1]), ([200, 7, 64], [131, 7, 1])],
                         ids=["few-rows", "many-rows"])
@pytest.mark.parametrize("n_q,n_kv,D", [(4, 2, 16), (5, 1, 48), (8, 8, 128), (3, 3, 80), (5, 1, 64)])
def test_qk_norm_rope_cache(dtype, n_q, n_kv, D, lengths, counts):
    """Few rows and many rows take different shapes of the bfloat16 kernel (one head or
    several heads per warp; 5 + 2 heads leave a last group that is not full)."""
    from thing_htn_2026_b200.config.base import PartSpec
    from thing_htn_2026_b200.parts import Runtime, part_class
    o = ops()
    fix = PagedFixture(n_kv, D, lengths, dtype)
    # the sequences already hold lengths - counts tokens
    old = [n - c for n, c in zip(lengths, counts)]
    keep = fix.slots
    fix.slots = [s for s, n in zip(keep, old) if n]
    rows, _ = fix.rows([n for n in old if n])
    fix.advance(rows, [n for n in old if n])
    fix.slots = keep
    before = fix.kv.storage.clone()

    rows, cu = fix.rows(counts)
    theta, eps = 12345.0, 1e-5
    rope = part_class("position", "rope")(PartSpec("rope", {"head_dim": D, "theta": theta}),
                                          Runtime(dtype, torch.device(DEV), {}))
    rope.ensure(256)
    qkv = rand((cu[-1], (n_q + 2 * n_kv) * D), dtype, 20, 2.0)
    qg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(21))).to(dtype)
    kg = (1 + 0.3 * torch.randn(D, generator=torch.Generator().manual_seed(22))).to(dtype)
    err = o.new_error_word(DEV)
    q = o.qk_norm_rope_cache(qkv.to(DEV), qg.to(DEV), kg.to(DEV), eps, rope.tables(), rows, fix.kv, n_q, True, err)
    assert int(err.item()) == 0

    positions = torch.cat([torch.arange(n - c, n) for n, c in zip(lengths, counts)])
    cos, sin = plain.rope_cos_sin(positions, D, theta, dtype)
    q_in = qkv[:, :n_q * D].reshape(-1, n_q, D)
    k_in = qkv[:, n_q * D:(n_q + n_kv) * D].reshape(-1, n_kv, D)
    v_in = qkv[:, (n_q + n_kv) * D:].reshape(-1, n_kv, D)
    q_want = plain.apply_rope(plain.rms_norm(q_in, qg, eps, dtype), cos, sin, dtype)
    k_want = plain.apply_rope(plain.rms_norm(k_in, kg, eps, dtype), cos, sin, dtype)
    close(q.reshape(-1, n_q, D), q_want, dtype, "q norm + rope")

    storage = fix.kv.storage.cpu()
    table = fix.kv.block_table.cpu()
    touched = torch.zeros_like(storage, dtype=torch.bool)
    row = 0
    for i, (n, c) in enumerate(zip(lengths, counts)):
        for p in range(n - c, n):
            page = int(table[fix.slots[i], p // 64])
            assert page >= 0
            close(storage[page, 0, :, p % 64], k_want[row], dtype, "k in cache")
            assert torch.equal(storage[page, 1, :, p % 64], v_in[row]), "v must be copied untouched"
            touched[page, :, :, p % 64] = True
            row += 1
    assert torch.equal(storage[~touched], before.cpu()[~touched]), "a cache place outside the step was written"


# ----------------------------------------------------------------------------- token choice


def test_argmax_lowest_index_on_ties():
    logits = torch.zeros(5, 1000)
    logits[0, [7, 500, 999]] = 3.0
    logits[1, 999] = 1.0
    logits[2] = -5.0                     # all equal: index 0
    logits[3, 0] = 9.0
    logits[4, [998, 999]] = 2.0
    out = ops().choose_tokens(logits.to(DEV)).cpu().tolist()
    assert out == [7, 999, 0, 0, 998]


@pytest.mark.parametrize("vocab", [300, 4097, 151936])
def test_sampling_matches_plain_draws(vocab):
    rows = 6
    logits = rand((rows, vocab), torch.float32, 30, 2.0)
    temperature = torch.tensor([0.7, 0.0, 1.0, 1.5, 0.3, 1.0])
    seed = torch.tensor([1, 2, 3, 2 ** 40 + 5, 7, 3], dtype=torch.int64)
    stream = torch.tensor([0, 1, 2, 3, 4, 2], dtype=torch.int32)
    step = torch.tensor([0, 5, 9, 1000, 2, 10], dtype=torch.int32)
    out = ops().choose_tokens(logits.to(DEV), temperature.to(DEV), seed.to(DEV), stream.to(DEV), step.to(DEV))
    for r in range(rows):
        want = plain.sample(logits[r].numpy(), float(temperature[r]), int(seed[r]), int(stream[r]), int(step[r]))
        assert int(out[r]) == want, f"row {r}"


def test_sampling_follows_the_distribution():
    """4000 draws from a 6-way distribution at temperature 0.8 against softmax(logits / 0.8)."""
    logits = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0, 1.5]])
    n = 4000
    batch = logits.repeat(n, 1).to(DEV)
    out = ops().choose_tokens(batch, torch.full((n,), 0.8, device=DEV), torch.full((n,), 99, dtype=torch.int64, device=DEV),
                              torch.zeros(n, dtype=torch.int32, device=DEV),
                              torch.arange(n, dtype=torch.int32, device=DEV)).cpu()
    freq = torch.bincount(out.long(), minlength=6).float() / n
    want = torch.softmax(logits[0] / 0.8, dim=0)
    assert (freq - want).abs().max() < 4 * (want * (1 - want) / n).sqrt().max() + 1e-3
