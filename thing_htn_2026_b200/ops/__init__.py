"""Python faces of the CUDA kernels.  Every function here takes CUDA tensors and launches
on the current stream; there is no CPU path.  Matrix products of the bfloat16 path may
go to the vendor library, as the reference's do (engine/engine.py:341-350); everything
else, and every product of the 32-bit path, is this library's own kernel.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import library
from .library import KernelLibraryError

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

# device error word bits (csrc/common.cuh)
ERR_TOKEN_RANGE, ERR_PAGE_UNMAPPED, ERR_POSITION_RANGE, ERR_WAIT_TIMEOUT = 1, 2, 4, 8
_ERR_TEXT = {
    ERR_TOKEN_RANGE: "a token id outside the vocabulary",
    ERR_PAGE_UNMAPPED: "a cache position whose page is not mapped",
    ERR_POSITION_RANGE: "a position beyond the rotary table",
    ERR_WAIT_TIMEOUT: "a bounded wait inside a kernel gave up",
}


class KernelError(RuntimeError):
    """A launcher refused its arguments, or a kernel reported a fault."""


_SIGNATURES = {
    "thn_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "thn_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_gemm_tcgen05_supported": [c_int, c_int, c_int],
    "thn_gemm_tcgen05_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_gemm_stream_supported": [c_int, c_int, c_int],
    "thn_gemm_stream_scratch": [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_gemm_stream_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_void_p, c_void_p],
    "thn_step_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_advance": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_qk_norm_rope_cache": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                               c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_int, c_void_p, c_void_p],
    "thn_attention_decode_fused_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_void_p, c_int,
                                        c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_int,
                                        c_void_p, c_void_p],
    "thn_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p],
    "thn_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "thn_scatter_i32": [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "thn_choose_tokens": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "thn_gather_i32": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "thn_attention_mma_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_fused_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_prefill_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "thn_attention_decode_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_int,
                                  c_void_p, c_void_p],
    "thn_attention_decode_blocks_per_sm": [c_int],
    "thn_attention_decode_cluster_splits": [],
    "thn_attention_decode_one_wave_splits": [c_int, c_int, c_int],
    "thn_attention_prefill_tile_rows": [],
    "thn_attention_decode_last_variant": [],
    "thn_attention_decode_streams": [],
    "thn_attention_tcgen05_supported": [c_int, c_int, c_int, c_int],
    "thn_attention_tcgen05_test_skip_loads": [c_int],
    "thn_attention_prefill_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                      c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                      c_int, c_void_p, c_void_p],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        loaded = library.load()
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        loaded.thn_set_pdl.argtypes = [c_int]
        loaded.thn_set_pdl.restype = None
        loaded.thn_set_pdl(0 if os.environ.get("THN_PDL", "1").strip().lower() in ("0", "false", "no", "off") else 1)
        loaded.thn_set_stream_early.argtypes = [c_int]
        loaded.thn_set_stream_early.restype = None
        if os.environ.get("THN_STREAM_EARLY"):
            loaded.thn_set_stream_early(int(os.environ["THN_STREAM_EARLY"]))
        loaded.thn_set_decode_cluster.argtypes = [c_int]
        loaded.thn_set_decode_cluster.restype = None
        loaded.thn_set_decode_cluster(0 if os.environ.get("THN_DECODE_CLUSTER", "1").strip() in ("0", "false", "off") else 1)
        loaded.thn_set_decode_stream_order.argtypes = [c_int]
        loaded.thn_set_decode_stream_order.restype = None
        loaded.thn_set_decode_stream_order(int(os.environ.get("THN_DECODE_STREAM_BY_LENGTH", 1)))
        loaded.thn_set_decode_stream.argtypes = [c_int, c_int]
        loaded.thn_set_decode_stream.restype = None
        loaded.thn_set_decode_stream(int(os.environ.get("THN_DECODE_STREAM", 1)),
                                     int(os.environ.get("THN_DECODE_STREAM_STAGES", 3)))
        loaded.thn_choose_tokens_scratch_floats.argtypes = [c_int, c_int]
        loaded.thn_choose_tokens_scratch_floats.restype = c_longlong
        loaded.thn_attention_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int]
        loaded.thn_attention_decode_scratch_floats.restype = c_longlong
        _lib = loaded
    return _lib


_sm_count = {}
launch_count = 0   # kernels of this library launched (or recorded into a graph) so far
calls_by_entry: Dict[str, int] = {}    # the same, per entry point of the kernel library


def _call(name: str, *args) -> None:
    global launch_count
    launch_count += 1
    calls_by_entry[name] = calls_by_entry.get(name, 0) + 1
    code = getattr(lib(), name)(*args)
    if code:
        raise KernelError(f"{name}: {lib().thn_last_error().decode()} (status {code})")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, what: str, dtype=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; this library runs on CUDA only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def new_error_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def raise_on_device_error(err: torch.Tensor, where: str) -> None:
    """Reads the error word (a synchronising copy) and raises if a kernel set a bit."""
    bits = int(err.item())
    if bits:
        err.zero_()
        reasons = [text for bit, text in _ERR_TEXT.items() if bits & bit]
        raise KernelError(f"{where}: device reported " + "; ".join(reasons))


# ------------------------------------------------------------------ rows and lengths


@dataclass
class StepRows:
    """Per-row indices of a packed step: the slot of each row's sequence and the row's
    absolute position; plus the batch description they were made from."""

    row_slot: torch.Tensor   # int32 [rows]
    row_pos: torch.Tensor    # int32 [rows]
    slots: torch.Tensor      # int32 [seqs]
    cu_seqlens: torch.Tensor  # int32 [seqs + 1]
    n_rows: int
    n_seqs: int
    max_q_len: int           # longest run of rows of one sequence (host knowledge)
    # Host knowledge: the most keys a row of this step may see (an upper bound; None: unknown).
    # Kernels may divide their work by it, which changes a result by rounding at most.  A step
    # captured as a graph is replayed only while its bound holds (see context_class).
    max_context: Optional[int] = None
    # Host knowledge: False if the sequences of the step hold about the same number of keys (see
    # lengths_differ); None: unknown.  Like max_context a hint that changes no result.
    lengths_differ: Optional[bool] = None


LONG_CONTEXT = 8192     # keys; a single-token step of few long sequences divides each key range further
CONTEXT_CLASS_BASE = 1024   # keys; the first class of context length ends below it
STREAM_MIN_CONTEXT = 1024   # keys from which many unsplit sequences go to the streaming decode attention


def context_class(longest: int) -> Tuple[int, int]:
    """(class, bound) of a step whose longest sequence holds ``longest`` keys: class 0 below
    CONTEXT_CLASS_BASE, then one class per doubling.  Steps of one class make the same choices,
    so one captured graph serves them; ``bound`` is the class's ``max_context``."""
    k = (max(0, int(longest)) // CONTEXT_CLASS_BASE).bit_length()
    return k, (CONTEXT_CLASS_BASE << k) - 1


def lengths_differ(lengths) -> bool:
    """Whether the shortest of the sequences is more than a quarter shorter than the longest:
    the class of a step, beside ``context_class``, by which a captured graph is chosen."""
    longest = max(lengths)
    return (longest - min(lengths)) * 4 > longest


def step_rows(cu_seqlens: torch.Tensor, slots: torch.Tensor, seq_lens: torch.Tensor, n_rows: int,
              max_q_len: int, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
              max_context: Optional[int] = None, lengths_differ: Optional[bool] = None) -> StepRows:
    _need(cu_seqlens, "step_rows cu_seqlens", torch.int32)
    _need(slots, "step_rows slots", torch.int32)
    _need(seq_lens, "step_rows seq_lens", torch.int32)
    n_seqs = slots.shape[0]
    if out is None:
        row_slot = torch.empty(n_rows, dtype=torch.int32, device=slots.device)
        row_pos = torch.empty(n_rows, dtype=torch.int32, device=slots.device)
    else:
        row_slot, row_pos = out
    _call("thn_step_rows", _ptr(row_slot), _ptr(row_pos), _ptr(cu_seqlens), _ptr(slots), _ptr(seq_lens), n_seqs,
          _stream())
    return StepRows(row_slot, row_pos, slots, cu_seqlens, n_rows, n_seqs, max_q_len, max_context=max_context,
                    lengths_differ=lengths_differ)


def advance(seq_lens: torch.Tensor, slots: torch.Tensor, cu_seqlens: torch.Tensor) -> None:
    _call("thn_advance", _ptr(_need(seq_lens, "advance seq_lens", torch.int32)), _ptr(slots), _ptr(cu_seqlens),
          slots.shape[0], _stream())


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> None:
    """dst.view(-1)[index[i]] = value[i]; index int64, value int32, all on the device."""
    _need(dst, "scatter_i32 dst", torch.int32)
    _need(index, "scatter_i32 index", torch.int64)
    _need(value, "scatter_i32 value", torch.int32)
    _call("thn_scatter_i32", _ptr(dst), _ptr(index), _ptr(value), index.shape[0], dst.numel(), _stream())


# ------------------------------------------------------------------ elementwise


def gather_rows(table: torch.Tensor, index: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m] = table[index[m]]; an index outside the table sets ERR_TOKEN_RANGE."""
    _need(table, "gather_rows table")
    _need(index, "gather_rows index", torch.int32)
    out = torch.empty((index.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    _call("thn_gather_rows", _ptr(out), _ptr(table), _ptr(index), index.shape[0], table.shape[1], table.shape[0],
          _code(table, "gather_rows"), _ptr(err), _stream())
    return out


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    _need(x, "rmsnorm x")
    _need(gain, "rmsnorm gain")
    if gain.shape[0] != x.shape[-1]:
        raise KernelError(f"rmsnorm: gain has {gain.shape[0]} entries, rows have {x.shape[-1]}")
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    _call("thn_rmsnorm", _ptr(y), _ptr(x), None, _ptr(gain), rows, x.shape[-1], float(eps),
          _code(x, "rmsnorm"), _code(gain, "rmsnorm gain"), _stream())
    return y


def add_rmsnorm(h: torch.Tensor, d: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """h <- round(h + d) in place; returns RMSNorm(h) * gain."""
    _need(h, "add_rmsnorm h")
    _need(d, "add_rmsnorm d", h.dtype)
    _need(gain, "add_rmsnorm gain")
    if tuple(d.shape) != tuple(h.shape) or gain.shape[0] != h.shape[-1]:
        raise KernelError(f"add_rmsnorm: shapes h {tuple(h.shape)}, d {tuple(d.shape)}, gain {tuple(gain.shape)}")
    y = torch.empty_like(h)
    rows = h.numel() // h.shape[-1]
    _call("thn_rmsnorm", _ptr(y), _ptr(h), _ptr(d), _ptr(gain), rows, h.shape[-1], float(eps),
          _code(h, "add_rmsnorm"), _code(gain, "add_rmsnorm gain"), _stream())
    return y


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """gu [rows, 2*I] (gate columns first) -> silu(gate) * up, [rows, I]."""
    _need(gu, "swiglu")
    rows, width = gu.shape
    if width % 2:
        raise KernelError(f"swiglu: width {width} is odd")
    out = torch.empty((rows, width // 2), dtype=gu.dtype, device=gu.device)
    _call("thn_swiglu", _ptr(out), _ptr(gu), rows, width // 2, _code(gu, "swiglu"), _stream())
    return out


def rope_table(cos: torch.Tensor, sin: torch.Tensor, inv_freq: torch.Tensor, first: int, count: int) -> None:
    _need(cos, "rope_table cos", torch.float32)
    _need(sin, "rope_table sin", torch.float32)
    _need(inv_freq, "rope_table inv_freq", torch.float32)
    if first + count > cos.shape[0]:
        raise KernelError(f"rope_table: rows [{first}, {first + count}) exceed the table of {cos.shape[0]}")
    _call("thn_rope_table", _ptr(cos), _ptr(sin), _ptr(inv_freq), first, count, inv_freq.shape[0], _stream())


# ------------------------------------------------------------------ matrix products


def _sm_count_of(device) -> int:
    index = torch.device(device).index or 0
    if index not in _sm_count:
        _sm_count[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_count[index]


# Products with at most STREAM_MAX_ROWS rows go to this library's weight-streaming kernel where it
# beats the vendor library (kernel_bench.py on B200, 1 to 16 rows, at the layer sizes of Qwen3-4B,
# -8B and -14B): a weight of at most STREAM_MAX_N rows (so few 128-row tiles that a cluster of
# four or more blocks shares each) under a reduction at least STREAM_MIN_K deep: o and down at
# 2560 x 4096, 2560 x 9728, 4096 x 4096, 4096 x 12288 (7.1 vs 10.3, 12.0 vs 20.4, 9.2 vs 12.2,
# 19.7 vs 31.3 us at 8 rows); and a weight of at least STREAM_MIN_N rows (the head: 123 vs 127,
# 191 vs 205, 233 vs 255 us).  The library wins on q/k/v and gate-up at every size (7.5 vs 10.0,
# 17.5 vs 21.0, 10.9 vs 13.2, 34.4 vs 36.8, 13.8 vs 16.7, 58.0 vs 59.5 us) and at 5120 x 5120 and
# 5120 x 17408 (11.5 vs 12.5, 31.2 vs 32.7 us).  The row limit comes from whole decode steps of
# the Qwen3-4B sizes, where a product also gains from starting under its predecessor's tail: with
# the streaming product a step of 17 / 24 / 32 / 33 / 48 / 64 rows takes 2.49 / 2.61 / 2.74 / 2.78 /
# 3.09 / 3.49 ms, with the library's 2.63 / 2.74 / 2.85 / 2.85 / 3.13 / 3.47 ms.
STREAM_MAX_ROWS = 48
STREAM_MIN_K = int(os.environ.get("THN_STREAM_MIN_K", 4096))
STREAM_MAX_N = int(os.environ.get("THN_STREAM_MAX_N", 4096))
STREAM_MIN_N = 65536
STREAM_POLICY = os.environ.get("THN_LINEAR_STREAM", "auto")     # auto | all | none (measurement)

_device_counters = {}


COUNTER_SLOTS = 1 << 20


def _counter_buffer(n: int, device) -> torch.Tensor:
    """Arrival counters for kernels whose last-arriving block finishes a shared result; zero
    between calls (the kernels reset them).  One buffer per device for the life of the
    process: captured graphs hold its address, so it is never replaced by a larger one."""
    if n > COUNTER_SLOTS:
        raise KernelError(f"a kernel asks for {n} arrival counters, the buffer holds {COUNTER_SLOTS}")
    index = torch.device(device).index or 0
    have = _device_counters.get(index)
    if have is None:
        have = torch.zeros(COUNTER_SLOTS, dtype=torch.int32, device=device)
        _device_counters[index] = have
    return have


_stream_needs = {}


def _stream_need(m: int, n: int, k: int, swiglu: bool, n_blocks: int):
    key = (m, n, k, swiglu, n_blocks)
    if key not in _stream_needs:
        floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
        lib().thn_gemm_stream_scratch(m, n, k, int(swiglu), n_blocks, ctypes.byref(floats), ctypes.byref(counters))
        _stream_needs[key] = (floats.value, counters.value)
    return _stream_needs[key]


def linear_stream(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                  swiglu: bool = False, err: Optional[torch.Tensor] = None, n_blocks: int = 0) -> torch.Tensor:
    """The TMA / tcgen05 weight-streaming product for steps of at most 64 rows (bfloat16
    operands, K a multiple of 8) -> ``[M, N]`` in bfloat16 or float32.  With ``swiglu`` the
    weight is ``[2 * I, K]`` (gate rows, then up rows) and the result is ``silu(gate) * up``,
    ``[M, I]``, in one kernel.  ``n_blocks`` overrides how the work is cut (tests): that many
    blocks with balanced runs, or, negative, one thread-block cluster of that size per tile."""
    _need(x, "linear_stream x", torch.bfloat16)
    _need(weight, "linear_stream weight", torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    if weight.shape[1] != k or (swiglu and weight.shape[0] % 2):
        raise KernelError(f"linear_stream: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    floats, n_counters = _stream_need(m, n, k, swiglu, n_blocks)
    counters = _counter_buffer(n_counters, x.device)
    scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _call("thn_gemm_stream_bf16", _ptr(out), DTYPE_CODE[out_dtype], _ptr(scratch), _ptr(counters), _ptr(x),
          _ptr(weight), m, n, k, int(swiglu), n_blocks, _ptr(err), _stream())
    return out


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, err: Optional[torch.Tensor] = None,
                   swiglu: bool = False) -> torch.Tensor:
    """The tcgen05 / TMEM / TMA product for steps with many rows: ``x [M, K] @ weight[N, K]^T``
    in bfloat16.  With ``swiglu`` the weight is ``[2 * I, K]`` (gate rows, then up rows) and the
    result is ``silu(gate) * up``, ``[M, I]``, in one kernel."""
    _need(x, "linear_tcgen05 x", torch.bfloat16)
    _need(weight, "linear_tcgen05 weight", torch.bfloat16)
    m, k = x.shape
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear_tcgen05: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    _call("thn_gemm_tcgen05_bf16", _ptr(out), _ptr(x), _ptr(weight), m, n, k, int(swiglu), _ptr(err), _stream())
    return out


def _stream_takes(m: int, n: int, k: int, fused: bool = False) -> bool:
    if STREAM_POLICY == "none" or not lib().thn_gemm_stream_supported(m, n, k):
        return False
    if STREAM_POLICY == "all":
        return True
    return not fused and m <= STREAM_MAX_ROWS and ((k >= STREAM_MIN_K and n <= STREAM_MAX_N) or n >= STREAM_MIN_N)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) for ``w_gate_up = cat(gate, up)``: one kernel where the
    weight-streaming product takes the shape, else the product followed by the activation."""
    if x.dtype == torch.bfloat16 and _stream_takes(x.shape[0], w_gate_up.shape[0] // 2, x.shape[1], fused=True):
        return linear_stream(x, w_gate_up, swiglu=True, err=err)
    return swiglu(linear(x, w_gate_up, err=err))


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           err: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [M, K] @ weight[N, K]^T.  float32: this library's FFMA kernel.  bfloat16 with few
    rows and a deep reduction or a tall weight: this library's weight-streaming kernel
    (``err``: the step's device error word for its bounded waits).  bfloat16 otherwise: the
    vendor library's tensor-core product with float32 accumulation (the reference's choice,
    engine/engine.py:341-350).  ``out_dtype=torch.float32`` keeps the accumulator's
    precision (used for logits)."""
    _need(x, "linear x")
    _need(weight, "linear weight", x.dtype)
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise KernelError(f"linear: shapes x {tuple(x.shape)}, weight {tuple(weight.shape)}")
    if x.dtype == torch.float32:
        out = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=x.device)
        _call("thn_gemm_f32", _ptr(out), _ptr(x), _ptr(weight), x.shape[0], weight.shape[0], x.shape[1], _stream())
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: dtype {x.dtype} is not supported")
    if _stream_takes(x.shape[0], weight.shape[0], x.shape[1]):
        return linear_stream(x, weight, out_dtype or torch.bfloat16, err=err)
    if out_dtype in (None, torch.bfloat16):
        return torch.nn.functional.linear(x, weight)
    return torch.mm(x, weight.t(), out_dtype=out_dtype)


# ------------------------------------------------------------------ attention


@dataclass
class KVView:
    """One cache entry as the kernels see it."""

    storage: torch.Tensor       # [pages, 2, n_kv, page_size, head_dim] of this entry
    block_table: torch.Tensor   # int32 [max_slots, max_pages_per_seq]
    n_kv: int
    page_size: int
    head_dim: int


@dataclass
class RowTiles:
    """Tiles of at most ``size`` consecutive rows of one sequence, for the prompt attention
    kernels: first packed row and row count of each tile (int32, on the device).  The
    kernels start at the end of the list, so it is ordered by the keys a tile sees,
    fewest first (see :func:`row_tiles_of`)."""

    row0: torch.Tensor
    rows: torch.Tensor
    n: int
    size: int


def row_tiles_of(counts, held, size: int):
    """Host lists (row0, rows) of the tiles of a step whose sequences bring ``counts[i]``
    rows on top of ``held[i]`` cached tokens, fewest keys first."""
    tiles, start = [], 0
    for c, h in zip(counts, held):
        for r in range(0, c, size):
            n = min(size, c - r)
            tiles.append((h + r + n, start + r, n))
        start += c
    tiles.sort()
    return [t[1] for t in tiles], [t[2] for t in tiles]


@dataclass
class RotaryTables:
    cos: torch.Tensor   # float32 [positions, rotary_dim / 2]
    sin: torch.Tensor
    rotary_dim: int


def qk_norm_rope_cache(qkv, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor],
                       eps: float, rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_q: int,
                       write_cache: bool, err: torch.Tensor) -> torch.Tensor:
    """qkv -> q, normalised and rotated; K and V go to the cache."""
    width = (n_q + 2 * kv.n_kv) * kv.head_dim
    if tuple(qkv.shape) != (rows.n_rows, width):
        raise KernelError(f"qk_norm_rope_cache: qkv is {tuple(qkv.shape)}, expected {(rows.n_rows, width)}")
    if kv.storage.dtype != qkv.dtype:
        raise KernelError(f"qk_norm_rope_cache: cache is {kv.storage.dtype}, activations {qkv.dtype}")
    _need(qkv, "qk_norm_rope_cache qkv")
    q = torch.empty((rows.n_rows, n_q * kv.head_dim), dtype=qkv.dtype, device=kv.storage.device)
    w_code = _code(q_gain, "qk gains") if q_gain is not None else DTYPE_CODE[qkv.dtype]
    _call("thn_qk_norm_rope_cache", _ptr(q), _ptr(qkv), _ptr(q_gain), _ptr(k_gain), w_code, float(eps),
          _ptr(rotary.cos) if rotary else None, _ptr(rotary.sin) if rotary else None,
          rotary.cos.shape[0] if rotary else 0, rotary.rotary_dim if rotary else 0,
          _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, rows.n_rows, n_q, int(write_cache),
          DTYPE_CODE[qkv.dtype], _ptr(err), _stream())
    return q


def attention_generic(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float,
                      window: Optional[int], err: torch.Tensor) -> torch.Tensor:
    _need(q, "attention q")
    out = torch.empty_like(q)
    _call("thn_attention_generic", _ptr(out), _ptr(q), _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage),
          _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, rows.n_rows, n_q,
          float(scale), int(window or 0), _code(q, "attention"), _ptr(err), _stream())
    return out


def prompt_attention_tile(dtype: torch.dtype, kv_head_dim: int, page_size: int, n_q: int, n_kv: int) -> int:
    """Rows per tile that the prompt attention kernel for these sizes works on, or 0 if the
    sizes go to the kernel that needs no tiles."""
    if dtype == torch.bfloat16 and lib().thn_attention_mma_supported(kv_head_dim, page_size, n_q, n_kv):
        return lib().thn_attention_prefill_tile_rows()
    return 0


def attention(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float, window: Optional[int],
              err: torch.Tensor, tiles: Optional[RowTiles] = None) -> torch.Tensor:
    """Causal attention of the step's rows over the cache (which already holds the step's
    own keys).  Chooses the kernel by dtype, head size and step shape; the tensor-core
    kernels for steps of several tokens per sequence need ``tiles``."""
    if q.dtype == torch.bfloat16 and lib().thn_attention_mma_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv):
        if rows.max_q_len == 1:
            return attention_decode_bf16(q, rows, kv, n_q, scale, window, err)
        if tiles is not None:
            if USE_TCGEN05_ATTENTION and lib().thn_attention_tcgen05_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv):
                return attention_prefill_tcgen05(q, rows, tiles, kv, n_q, scale, window, err)
            return attention_prefill_bf16(q, rows, tiles, kv, n_q, scale, window, err)
    return attention_generic(q, rows, kv, n_q, scale, window, err)


def attention_prefill_tcgen05(q: torch.Tensor, rows: StepRows, tiles: RowTiles, kv: KVView, n_q: int, scale: float,
                              window: Optional[int], err: torch.Tensor) -> torch.Tensor:
    """tcgen05 / TMEM / TMA flash attention for steps with several tokens per sequence
    (bfloat16, head size 128)."""
    _need(q, "attention q", torch.bfloat16)
    out = torch.empty_like(q)
    _check_tiles(tiles)
    _call("thn_attention_prefill_tcgen05", _ptr(out), _ptr(q), _ptr(tiles.row0), _ptr(tiles.rows),
          tiles.n, q.shape[0], _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), kv.storage.shape[0],
          _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_q, float(scale),
          int(window or 0), _ptr(err), _stream())
    return out


USE_TCGEN05_ATTENTION = os.environ.get("THN_ATTN_TCGEN05", "1").strip().lower() not in ("0", "false", "no", "off")


def ROW_TILE() -> int:
    """Rows per tile that the tensor-core prompt attention kernels work on."""
    return lib().thn_attention_prefill_tile_rows()


def _check_tiles(tiles: RowTiles) -> None:
    if tiles.size != ROW_TILE():
        raise KernelError(f"prompt attention: row tiles of {tiles.size} rows, the kernel works on {ROW_TILE()}")
    _need(tiles.row0, "row tiles", torch.int32)
    _need(tiles.rows, "row tiles", torch.int32)


def attention_prefill_bf16(q: torch.Tensor, rows: StepRows, tiles: RowTiles, kv: KVView, n_q: int, scale: float,
                           window: Optional[int], err: torch.Tensor) -> torch.Tensor:
    """Tensor-core flash attention for steps with several tokens per sequence."""
    _need(q, "attention q", torch.bfloat16)
    out = torch.empty_like(q)
    _check_tiles(tiles)
    _call("thn_attention_prefill_bf16", _ptr(out), _ptr(q), _ptr(tiles.row0), _ptr(tiles.rows),
          tiles.n, _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_q, float(scale), int(window or 0),
          _ptr(err), _stream())
    return out


DECODE_MAX_SPLITS = 32     # the splits of a key range are combined by the lanes of one warp


def decode_splits(n_seqs: int, n_kv: int, device, head_dim: int = 128, fused: bool = False,
                  context: Optional[int] = None, differ: Optional[bool] = None) -> int:
    """Splits of the key range per (sequence, kv head) of a single-token step: as many as fill
    the SMs once, the splits of a pair being the blocks of one thread-block cluster (at most
    eight, six unless the pairs are very few), all clusters resident at once.  It depends on the
    batch and on ``context`` (the step's ``max_context``, a bound that holds for every replay of
    a captured step), never on the lengths themselves."""
    if os.environ.get("THN_DECODE_SPLITS"):
        return int(os.environ["THN_DECODE_SPLITS"])
    pairs = max(1, n_seqs * n_kv)
    if long_sequences_stream(n_seqs, n_kv, context, differ, device):
        return 1           # unsplit: the streaming kernel's step
    one_wave = lib().thn_attention_decode_one_wave_splits(head_dim, int(fused), pairs)
    if context is not None and context >= LONG_CONTEXT:
        # Few long sequences: a block works through its tiles one after the other, and a cluster's
        # blocks are too few to draw the memory bandwidth.  Two blocks per SM, meeting in global
        # memory, read 32,768 keys of one sequence in 33 us against 56 us (B200, 8 kv heads);
        # below 8,192 keys the cluster's cheaper merge wins.
        wide = min(DECODE_MAX_SPLITS, 2 * _sm_count_of(device) // pairs)
        if wide >= 2 * max(1, one_wave):
            return wide
    return max(1, one_wave)


def long_sequences_stream(n_seqs: int, n_kv: int, context: Optional[int], differ: Optional[bool], device) -> bool:
    """Whether a single-token step is one for the streaming decode attention by what the host
    knows: sequences that may hold STREAM_MIN_CONTEXT keys or more, about as many (sequence, kv
    head) pairs as SMs or more, and, if the lengths differ, at least two pairs per resident
    block, so that long and short ones can be paired (with one pair per block the longest
    sequence alone would set the time: 4.18 against 4.08 ms per step at batch 16 with 117 to
    2,026 keys, Qwen3-8B sizes).  Measured on B200, Qwen3-4B sizes, equal lengths, ms per step
    with one block or one cluster per pair against the streaming kernel: batch 16 / 24 / 32 / 48
    at 2,048 keys 3.03 / 3.51 / 3.87 / 4.90 against 2.98 / 3.36 / 3.78 / 4.64; at 4,096 keys
    3.85 / 4.76 / 5.42 / 7.46 against 3.69 / 4.38 / 5.18 / 6.75; level at 1,024 keys; batch 12
    and below: the cluster."""
    if context is None or context < STREAM_MIN_CONTEXT or not lib().thn_attention_decode_streams():
        return False
    pairs, sms = n_seqs * n_kv, _sm_count_of(device)
    if differ is not False:
        return pairs >= 4 * sms          # two blocks per SM, two pairs per block
    return pairs * 20 >= 17 * sms


def decode_hints(rows: StepRows, n_kv: int, n_splits: int, device) -> int:
    """What the host knows of a single-token step, as the kernels' ``hints`` bits: 1 unless the
    sequences are known to be about equally long; 2 if the step is unsplit and
    :func:`long_sequences_stream` says so."""
    hints = 0 if rows.lengths_differ is False else 1
    if n_splits == 1 and long_sequences_stream(rows.n_rows, n_kv, rows.max_context, rows.lengths_differ, device):
        hints |= 2
    return hints


def attention_decode_bf16(q: torch.Tensor, rows: StepRows, kv: KVView, n_q: int, scale: float,
                          window: Optional[int], err: torch.Tensor, n_splits: Optional[int] = None,
                          scratch: Optional[torch.Tensor] = None, fused_merge: bool = True) -> torch.Tensor:
    """Split-KV flash decoding: one token per sequence.  Partial results of the splits go
    through float32 scratch memory, which is allocated here unless given."""
    _need(q, "attention q", torch.bfloat16)
    n_seqs = rows.n_rows
    if n_splits is None:
        n_splits = decode_splits(n_seqs, kv.n_kv, q.device, kv.head_dim, context=rows.max_context,
                                 differ=rows.lengths_differ)
    need = lib().thn_attention_decode_scratch_floats(n_seqs, n_q, n_splits, kv.head_dim)
    if need and scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if need and scratch.numel() < need:
        raise KernelError(f"attention_decode: scratch has {scratch.numel()} floats, {need} needed")
    counters = _counter_buffer(n_seqs * kv.n_kv, q.device) if n_splits > 1 and fused_merge else None
    out = torch.empty_like(q)
    _call("thn_attention_decode_bf16", _ptr(out), _ptr(q), _ptr(rows.row_slot), _ptr(rows.row_pos),
          _ptr(kv.storage), _ptr(kv.block_table), kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim,
          n_seqs, n_q, n_splits, float(scale), int(window or 0), _ptr(scratch), _ptr(counters), kv.storage.shape[0],
          decode_hints(rows, kv.n_kv, n_splits, q.device), _ptr(err), _stream())
    return out


FUSE_DECODE_ATTENTION = os.environ.get("THN_FUSE_DECODE", "1").strip().lower() not in ("0", "false", "no", "off")


def qkv_attention(qkv: torch.Tensor, q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                  rotary: Optional[RotaryTables], rows: StepRows, kv: KVView, n_q: int, scale: float,
                  window: Optional[int], write_cache: bool, err: torch.Tensor,
                  tiles: Optional[RowTiles] = None) -> torch.Tensor:
    """From the raw q/k/v rows of a step to the attention output: per-head q/k norm, rotation,
    cache write and attention over the cache.  One kernel for single-token steps in bfloat16
    with head norm and full rotation at the tensor-core kernel's sizes; otherwise
    :func:`qk_norm_rope_cache` followed by :func:`attention`."""
    fusable = (FUSE_DECODE_ATTENTION and rows.max_q_len == 1
               and qkv.dtype == torch.bfloat16 and q_gain is not None and k_gain is not None and rotary is not None
               and rotary.rotary_dim == kv.head_dim and kv.storage.dtype == torch.bfloat16
               and lib().thn_attention_fused_supported(kv.head_dim, kv.page_size, n_q, kv.n_kv))
    if not fusable:
        q = qk_norm_rope_cache(qkv, q_gain, k_gain, eps, rotary, rows, kv, n_q, write_cache, err)
        return attention(q, rows, kv, n_q, scale, window, err, tiles)
    n_seqs = rows.n_rows
    width = (n_q + 2 * kv.n_kv) * kv.head_dim
    if tuple(qkv.shape) != (n_seqs, width):
        raise KernelError(f"qkv_attention: qkv is {tuple(qkv.shape)}, expected {(n_seqs, width)}")
    n_splits = decode_splits(n_seqs, kv.n_kv, qkv.device, kv.head_dim, fused=True, context=rows.max_context,
                             differ=rows.lengths_differ)
    need = lib().thn_attention_decode_scratch_floats(n_seqs, n_q, n_splits, kv.head_dim)
    scratch = torch.empty(need, dtype=torch.float32, device=qkv.device) if need else None
    counters = _counter_buffer(n_seqs * kv.n_kv, qkv.device) if n_splits > 1 else None
    out = torch.empty((n_seqs, n_q * kv.head_dim), dtype=torch.bfloat16, device=qkv.device)
    _call("thn_attention_decode_fused_bf16", _ptr(out), _ptr(qkv), _ptr(q_gain), _ptr(k_gain),
          _code(q_gain, "qk gains"), float(eps), _ptr(rotary.cos), _ptr(rotary.sin), rotary.cos.shape[0],
          int(bool(write_cache)), _ptr(rows.row_slot), _ptr(rows.row_pos), _ptr(kv.storage), _ptr(kv.block_table),
          kv.block_table.shape[1], kv.n_kv, kv.page_size, kv.head_dim, n_seqs, n_q, n_splits, float(scale),
          int(window or 0), _ptr(scratch), _ptr(counters), kv.storage.shape[0],
          decode_hints(rows, kv.n_kv, n_splits, qkv.device), _ptr(err), _stream())
    return out


# ------------------------------------------------------------------ token choice


def choose_tokens(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
                  seed: Optional[torch.Tensor] = None, stream_id: Optional[torch.Tensor] = None,
                  step: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                  slots: Optional[torch.Tensor] = None, last_token: Optional[torch.Tensor] = None,
                  bump_step: bool = False) -> torch.Tensor:
    """logits float32 [rows, vocab] -> int32 [rows].  Rows with temperature 0 (or no
    temperature tensor at all) take the argmax, lowest index on ties; others are drawn
    from softmax(logits / T) with Philox noise keyed by (seed, stream, step) of the row.
    With ``slots`` the per-row values are per-sequence state indexed by ``slots[row]``;
    ``last_token`` (same indexing) also receives the choice; ``bump_step`` increments the
    step counter after use."""
    _need(logits, "choose_tokens logits", torch.float32)
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
        _need(seed, "seed", torch.int64)
        _need(stream_id, "stream", torch.int32)
        _need(step, "step", torch.int32)
    need = lib().thn_choose_tokens_scratch_floats(rows, vocab)
    scratch = torch.empty(need, dtype=torch.float32, device=logits.device) if need else None
    _call("thn_choose_tokens", _ptr(out), _ptr(logits), rows, vocab, logits.stride(0), _ptr(temperature),
          _ptr(seed), _ptr(stream_id), _ptr(step), _ptr(slots), _ptr(last_token), int(bump_step), _ptr(scratch),
          _stream())
    return out


def gather_i32(src: torch.Tensor, index: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(src, "gather_i32 src", torch.int32)
    _need(index, "gather_i32 index", torch.int32)
    if out is None:
        out = torch.empty(index.shape[0], dtype=torch.int32, device=src.device)
    _call("thn_gather_i32", _ptr(out), _ptr(src), _ptr(index), index.shape[0], _stream())
    return out


__all__ = [
    "KernelError", "KernelLibraryError", "KVView", "RotaryTables", "RowTiles", "StepRows", "row_tiles_of", "prompt_attention_tile", "linear_stream", "linear_swiglu", "linear_tcgen05", "add_rmsnorm", "advance",
    "ROW_TILE", "attention", "attention_decode_bf16", "attention_generic", "attention_prefill_bf16", "attention_prefill_tcgen05", "decode_splits", "choose_tokens", "gather_i32", "gather_rows", "lib", "linear", "new_error_word",
    "qk_norm_rope_cache", "qkv_attention", "raise_on_device_error", "rmsnorm", "rope_table", "scatter_i32", "step_rows", "swiglu",
]
