"""The decode-attention entry point that allocates nothing.

A host that talks to the library through its C symbols may have no way to get scratch
memory at call time (all device memory already spoken for, or a thread that must not wait
on the driver's allocator).  ``thn_attention_decode_bf16_no_alloc`` serves such a host from
a fixed array inside the library.  This test calls it the way that host would, through the
exported symbol with raw pointers, twice in a row on different inputs (the second call finds
the first call's leftovers in the array), and compares each result with what the ordinary
entry point gives on the same inputs with scratch from the test.  It also checks that a
request larger than the array is refused before anything runs.

The file's name sorts last so that a run stopping at the first failure has already been
through every other test.  It must pass alone in a fresh process and after the others.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def c_symbol():
    from thing_htn_2026_b200.ops import library
    lib = ctypes.CDLL(library.build())
    fn = lib.thn_attention_decode_bf16_no_alloc
    v, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [v, v, v, v, v, v, i, i, i, i, i, i, i, f, i, v, v]
    fn.restype = i
    lib.thn_last_error.restype = ctypes.c_char_p
    return lib, fn


def make_case(n_seqs, n_q, n_kv, head_dim, lengths, seed):
    """A cache entry filled with random keys and values, and one query row per sequence
    whose own token is the last one of its sequence."""
    from thing_htn_2026_b200 import ops
    from thing_htn_2026_b200.cache import KVSpec, SequenceCache
    g = torch.Generator().manual_seed(seed)
    total = sum(-(-n // 64) * 64 for n in lengths)
    cache = SequenceCache([KVSpec(n_kv, head_dim)], max_tokens=total, dtype=torch.bfloat16, device=DEV,
                          max_slots=n_seqs)
    slots = cache.open(n_seqs)
    cache.prepare(slots, lengths)
    kv = cache.kv_view(0)
    kv.storage.copy_(torch.randn(kv.storage.shape, generator=g).to(torch.bfloat16))
    row_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    row_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    q = torch.randn((n_seqs, n_q * head_dim), generator=g).to(torch.bfloat16).to(DEV)
    rows = ops.StepRows(row_slot, row_pos, row_slot, torch.arange(n_seqs + 1, dtype=torch.int32, device=DEV),
                        n_seqs, n_seqs, 1)
    return cache, kv, rows, q


def test_no_alloc_entry_point_matches_the_ordinary_one():
    from thing_htn_2026_b200 import ops
    lib, no_alloc = c_symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row: the second is smaller and shaped differently, so whatever the first
    # left in the shared array lies around its partials
    cases = [dict(n_seqs=6, n_q=8, n_kv=2, head_dim=128, lengths=[700, 64, 65, 1, 333, 128], n_splits=5, window=0),
             dict(n_seqs=3, n_q=4, n_kv=2, head_dim=64, lengths=[90, 500, 17], n_splits=3, window=70)]
    for number, case in enumerate(cases):
        cache, kv, rows, q = make_case(case["n_seqs"], case["n_q"], case["n_kv"], case["head_dim"], case["lengths"],
                                       seed=number)
        scale = case["head_dim"] ** -0.5
        err = ops.new_error_word(DEV)
        want = ops.attention_decode_bf16(q, rows, kv, case["n_q"], scale, case["window"] or None, err,
                                         n_splits=case["n_splits"])
        got = torch.full_like(q, float("nan"))
        status = no_alloc(got.data_ptr(), q.data_ptr(), rows.row_slot.data_ptr(), rows.row_pos.data_ptr(),
                          kv.storage.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[1], kv.n_kv,
                          kv.page_size, kv.head_dim, case["n_seqs"], case["n_q"], case["n_splits"], scale,
                          case["window"], err.data_ptr(), stream)
        assert status == 0, lib.thn_last_error().decode()
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        bad = (got.float() - want.float()).abs() > 1e-2 + want.float().abs() / 64     # the kernel tests' rule
        assert not bad.any(), f"call {number}: {int(bad.sum())} values differ from the ordinary entry point"
        assert torch.isfinite(got.float()).all()


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    lib, no_alloc = c_symbol()
    # 512 sequences x 64 heads x 32 splits x (128 + 2) floats is far beyond the built-in array
    status = no_alloc(None, None, None, None, None, None, 1, 8, 64, 128, 512, 64, 32, 0.1, 0, None, None)
    assert status != 0
    message = lib.thn_last_error().decode()
    assert "floats of scratch" in message and "holds" in message
