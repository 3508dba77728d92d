"""Python face of the CUDA kernels: loads the shared library built from
``csrc/`` and wraps each exported entry point.  Every wrapper checks dtypes,
shapes and contiguity, launches on torch's current stream and raises on a launch
error.  There is no fallback: without a CUDA device or without the library these
functions raise.

Matrix products in bfloat16 go to the vendor library through ``torch.mm`` (the
reference's ``nn.Linear`` does the same, batchspec/models/modules/attention/base.py:32-39);
float32 products use this package's own FFMA kernel so that no reduced-precision
mode can slip in.
"""
from __future__ import annotations

import ctypes
import sys
import threading
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

import torch

_lib = None
_lock = threading.Lock()
_launches = 0          # kernels of this package launched (for the benchmark's count)

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}")


_SIGNATURES = {
    "bspec_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "bspec_add_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "bspec_gather_rows_add": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "bspec_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "bspec_rope_kv_append": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p],
    "bspec_rope_inplace": [c_void_p, c_int, c_int, c_longlong, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "bspec_attention_generic": [c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p],
    "bspec_attention_bf16": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong,
                             c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p],
    "bspec_gemm_tc_plan": [c_int, c_int, c_int, c_int, c_void_p],
    "bspec_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "bspec_gemm_tc_qkv_rope": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
                               c_void_p],
    "bspec_attention_prefill_tc": [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_longlong, c_int, c_int, c_int, c_int, c_int, c_float,
                                   c_int, c_int, c_void_p, c_void_p],
    "bspec_sgemm_tn": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
    "bspec_pick_slices": [c_int],
    "bspec_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "bspec_sample": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ulonglong, c_void_p,
                     c_void_p, c_void_p, c_void_p, c_void_p],
}


def load_library():
    """Load (building on first use) the kernel library.  Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from ..csrc.build import library_path
        path = library_path(build=True)
        lib = ctypes.CDLL(str(path))
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_longlong if name == "bspec_gemm_tc_plan" else c_int
        _lib = lib
        from . import debug
        debug.apply_environment(sys.modules[__name__], lib)
        global _BOUNDS_ACTIVE
        from ..csrc.build import bounds_requested
        _BOUNDS_ACTIVE = bounds_requested()
    return _lib


_BOUNDS_ACTIVE = False


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of the library (on by default)."""
    lib = load_library()
    lib.bspec_set_pdl.argtypes = [c_int]
    lib.bspec_set_pdl.restype = None
    lib.bspec_set_pdl(int(bool(on)))


_TRACE_SETTERS = ["bspec_trace_set_attention_tcgen05", "bspec_trace_set_elementwise", "bspec_trace_set_attention_generic", "bspec_trace_set_attention_bf16",
                  "bspec_trace_set_gemm_fp32", "bspec_trace_set_sampling", "bspec_trace_set_gemm_tcgen05"]
TRACE_KERNEL_NAMES = {1: "embed", 2: "add_rmsnorm", 3: "gather_rows_add", 4: "silu_mul", 5: "rope_kv_append",
                      6: "rope_inplace", 7: "attn_generic", 8: "attn_decode", 9: "attn_prefill", 10: "sgemm",
                      11: "sample_threshold", 12: "sample_pick", 13: "sample_final", 20: "gemm_tcgen05", 30: "attn_prefill_tc"}


def set_trace(buf: Optional[torch.Tensor], count: Optional[torch.Tensor]) -> None:
    """Tuning aid.  ``buf`` int64 [capacity, 3] and ``count`` int32 [2] = {0, capacity} on the device: from now on
    block 0 of every kernel appends (kernel id, start ns, ns at which its wait on the predecessor returned).
    ``None`` switches it off.  Set it before capturing a graph that should record."""
    lib = load_library()
    for name in _TRACE_SETTERS:
        fn = getattr(lib, name)
        fn.argtypes = [c_void_p, c_void_p]
        fn.restype = c_int
        _check(fn(_ptr(buf), _ptr(count)), name)


def library_file() -> str:
    load_library()
    from ..csrc.build import library_path
    return str(library_path(build=False))


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    """Account for kernels of this package launched by a CUDA-graph replay."""
    global _launches
    _launches += int(n)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("batchspec_b200 kernels run on a CUDA device only; got a tensor on " + str(t.device))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = [None]


def _stream() -> int:
    """Handle of torch's current stream on the current device.  Asked for at every launch (a graph capture
    switches streams), so through the one call that does nothing else."""
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index[0] is None:
        _device_index[0] = torch.cuda.current_device()
    return _raw_stream(_device_index[0])


def _check(err: int, name: str) -> None:
    global _launches
    _launches += 1
    if err != 0:
        raise KernelError(f"{name}: CUDA error {err}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------- rows

def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    _require_cuda(ids, table, out)
    assert ids.dtype == torch.int32 and out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous()
    n, d = out.shape
    assert table.shape[1] == d and ids.numel() == n
    _check(load_library().bspec_embed(ids.data_ptr(), table.data_ptr(), _dtype_code(table.dtype), out.data_ptr(),
                                      n, d, table.shape[0], float(scale), _stream()), "embed")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor) -> None:
    _require_cuda(resid, delta, weight, out)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and out.is_contiguous()
    n, d = resid.shape
    assert out.shape == resid.shape and weight.numel() == d
    if delta is not None:
        assert delta.shape == resid.shape and delta.is_contiguous()
    dd = _dtype_code(delta.dtype) if delta is not None else _dtype_code(out.dtype)
    _check(load_library().bspec_add_rmsnorm(resid.data_ptr(), _ptr(delta), dd, weight.data_ptr(),
                                            _dtype_code(weight.dtype), out.data_ptr(), _dtype_code(out.dtype),
                                            n, d, float(eps), _stream()), "add_rmsnorm")


def gather_rows_add(resid: torch.Tensor, pending: Optional[torch.Tensor], rows: torch.Tensor,
                    out: torch.Tensor) -> None:
    _require_cuda(resid, pending, rows, out)
    assert resid.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    assert resid.is_contiguous() and out.is_contiguous() and (pending is None or pending.is_contiguous())
    pd = _dtype_code(pending.dtype) if pending is not None else F32
    _check(load_library().bspec_gather_rows_add(resid.data_ptr(), _ptr(pending), pd, rows.data_ptr(), out.data_ptr(),
                                                out.shape[0], out.shape[1], resid.shape[0], _stream()),
           "gather_rows_add")


GLU_FUSION = True
GLU_GROUP = 8      # gate/up interleave of weights prepared for the fused epilogues: 8 gate rows, then their 8 up rows


def silu_mul(u: torch.Tensor, out: torch.Tensor, group: int = 0) -> None:
    """out = silu(gate) * up.  ``group`` 0: u = [gate | up]; G > 0: blocks of G gate columns and their G up columns."""
    _require_cuda(u, out)
    n, inter = out.shape
    assert u.shape == (n, 2 * inter) and u.dtype == out.dtype and u.is_contiguous() and out.is_contiguous()
    _check(load_library().bspec_silu_mul(u.data_ptr(), out.data_ptr(), _dtype_code(u.dtype), n, inter, int(group),
                                         _stream()), "silu_mul")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GLU_GROUP) -> torch.Tensor:
    """[I, d] gate and up rows -> [2I, d] in blocks of ``group`` gate rows followed by their up rows."""
    inter, d = gate.shape
    assert inter % group == 0 and up.shape == gate.shape
    return torch.stack([gate.view(inter // group, group, d), up.view(inter // group, group, d)], dim=1).reshape(2 * inter, d).contiguous()


def linear_glu(x: torch.Tensor, w13: torch.Tensor, group: int = GLU_GROUP) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for bfloat16 with ``w13`` interleaved by ``interleave_gate_up``: one kernel with the
    activation in the GEMM's epilogue for decode-sized steps, vendor GEMM + activation kernel otherwise."""
    _require_cuda(x, w13)
    M, K = x.shape
    N = w13.shape[0]
    inter = N // 2
    if (GLU_FUSION and x.dtype == torch.bfloat16 and K % 8 == 0 and M > 0 and group == GLU_GROUP
            and x.is_contiguous() and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        out = torch.empty((M, inter), dtype=x.dtype, device=x.device)
        _check(load_library().bspec_gemm_tc(x.data_ptr(), w13.data_ptr(), out.data_ptr(), M, N, K, 0, 1,
                                            _status_word(x.device).data_ptr(), sm_count(x.device), _stream()), "gemm_tc_glu")
        return out
    u = linear(x, w13)
    out = torch.empty((M, inter), dtype=x.dtype, device=x.device)
    silu_mul(u, out, group)
    return out


def rope_frequency_table(freqs: torch.Tensor, device) -> torch.Tensor:
    """The form in which the rotary kernels take their frequencies: float32 [2, n], the leading parts of the
    float64 values in row 0 and the remainders in row 1 (their sum is the float64 value to 2^-48).  The kernels
    form the angle position * frequency in float64 from it."""
    f = freqs.detach().to("cpu", torch.float64).reshape(-1)
    hi = f.to(torch.float32)
    lo = (f - hi.to(torch.float64)).to(torch.float32)
    return torch.stack([hi, lo]).contiguous().to(device)


def rope_kv_append(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                   inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, positions: torch.Tensor,
                   tok_entry: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor, cache: torch.Tensor,
                   page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and write k and v of every token into the cache
    page of its position.  ``inv_freq``: a ``rope_frequency_table`` of rotary_dim / 2 frequencies.
    ``cache``: one layer's pages, any shape with
    2 * n_kv_heads * page_size * head_dim elements per page, laid out
    [page][k|v][kv head][row][dim]."""
    _require_cuda(qkv, positions, cache)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert cache.dtype == qkv.dtype and cache.is_contiguous()
    assert positions.dtype == torch.int32 and tok_entry.dtype == torch.int32
    if rotary_dim:
        assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rotary_dim // 2) and inv_freq.is_contiguous()
    _check(load_library().bspec_rope_kv_append(
        qkv.data_ptr(), _dtype_code(qkv.dtype), n, n_heads, n_kv_heads, head_dim, _ptr(inv_freq), int(rotary_dim),
        int(bool(interleaved)), positions.data_ptr(), tok_entry.data_ptr(), kv_indptr.data_ptr(),
        kv_indices.data_ptr(), cache.data_ptr(), int(page_size), int(bool(write_kv)), cache.shape[0], _stream()),
        "rope_kv_append")


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int,
                 interleaved: bool = False) -> None:
    """x: [n, H, hd] view whose last two dims are dense; rows may be strided.  ``inv_freq``: a
    ``rope_frequency_table``."""
    _require_cuda(x, positions, inv_freq)
    n, H, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd and positions.dtype == torch.int32
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, rotary_dim // 2) and inv_freq.is_contiguous()
    _check(load_library().bspec_rope_inplace(x.data_ptr(), _dtype_code(x.dtype), n, x.stride(0), H, hd,
                                             inv_freq.data_ptr(), int(rotary_dim), int(bool(interleaved)),
                                             positions.data_ptr(), _stream()), "rope_inplace")


# ---------------------------------------------------------------------------- attention

# Which attention kernels may run; tests switch these to compare kernels with each other (see also kernels/debug.py)
USE_TMA_ATTENTION = True
USE_TC_ATTENTION = True         # tcgen05 kernel for long prompt portions
BALANCED_ATTENTION = True       # equal shares of key tiles over a fixed grid for decode
FORCE_GENERIC_ATTENTION = False      # tests set this to compare the tensor-core kernels with the generic one
_sm_counts = {}


def sm_count(device=None) -> int:
    """Number of SMs of ``device`` (default: the current one), asked once per device."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _sm_counts:
        _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return _sm_counts[idx]


_tile_counters = {}               # device -> zeroed int32 buffers kept alive (graphs hold their addresses)


def attention_splits(n_entries: int, n_kv_heads: int, group: int, max_q_len: int, max_kv_len: int,
                     ctas_per_sm: int = 3) -> int:
    """How many ways the split-key kernel cuts each request's keys.  Every CTA pays a prologue and, with more
    than one split, a join, so long chunks are preferred: if chunks of at least 128 keys give no more CTAs than
    fit on the device at once, use them all (small batches: fill the SMs); otherwise chunks of at least 512
    keys, one split if that already keeps four fifths of the last wave busy, else the count that wastes the
    least of it.  1 when the step also holds long portions (they go to the 64-row kernel, which fills the
    device by itself)."""
    short = max(1, 16 // group)
    if max_q_len > short:
        return 1
    row_tiles = -(-(max_q_len * group) // 16)
    base = max(1, n_entries * n_kv_heads * row_tiles)
    slots = sm_count() * ctas_per_sm
    fine = min(64, max(1, -(-max_kv_len // 128)))
    if base * fine <= slots:
        return fine
    eff = lambda s: (base * s) / (-(-(base * s) // slots) * slots)
    if eff(1) >= 0.8:
        return 1
    best, best_eff = 1, eff(1)
    for s in range(2, min(64, max(1, max_kv_len // 512)) + 1):
        if eff(s) > best_eff + 1e-9:
            best, best_eff = s, eff(s)
    return best


_work_counters = {}               # device -> two zeroed ints: the prompt attention kernel's item counter


def _work_counter(device) -> torch.Tensor:
    if device not in _work_counters:
        _work_counters[device] = torch.zeros((2,), dtype=torch.int32, device=device)
    return _work_counters[device]


def _counters(device, n: int) -> torch.Tensor:
    bufs = _tile_counters.setdefault(device, [])
    if not bufs or bufs[-1].numel() < n:
        bufs.append(torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device))
    return bufs[-1]


def _attention_plan(device, ctx, tables, n_heads: int, n_kv_heads: int, head_dim: int):
    """Which bfloat16 attention kernels a step launches for layers of these sizes, with their scratch and the
    addresses of the step's metadata (kept alive by ``ctx`` and ``tables``)."""
    group = n_heads // n_kv_heads
    short = max(1, 16 // group)
    # the TMA-fed split-key kernels (page sizes 8..64) fit two CTAs per SM, the plain one three
    tma = USE_TMA_ATTENTION and tables.page_size % 8 == 0 and 64 % tables.page_size == 0
    # Equal shares of all key tiles over a fixed grid (cut on the device from the step's lengths): n_splits is
    # then only the most partial results a row tile may be left in, and the scratch is indexed by request.
    balanced = int(tma and BALANCED_ATTENTION and ctx.n_entries <= 512 and not ctx.extras.get("attn_splits"))
    if balanced:
        n_splits = min(64, max(16, -(-4 * sm_count(device) // (ctx.n_entries * n_kv_heads)) + 2))
    else:
        n_splits = ctx.extras.get("attn_splits") or attention_splits(ctx.n_entries, n_kv_heads, group, ctx.max_q_len,
                                                                     ctx.max_kv_len, 2 if tma else 3)
    run_decode = int(ctx.extras.get("min_q_len", 1) <= short)
    run_prefill = int(ctx.max_q_len > short)
    o_part = ml_part = counters = None
    if n_splits > 1 and run_decode:
        rows = ctx.n_entries * min(ctx.max_q_len, short) if balanced else ctx.n_tokens
        o_part = torch.empty((rows * n_heads * n_splits * head_dim,), dtype=torch.float32, device=device)
        ml_part = torch.empty((rows * n_heads * n_splits * 2,), dtype=torch.float32, device=device)
        row_tiles = -(-(min(ctx.max_q_len, short) * group) // 16)
        counters = _counters(device, ctx.n_entries * n_kv_heads * row_tiles)
        ctx.extras[("attention scratch", n_heads, n_kv_heads, head_dim, id(tables))] = (o_part, ml_part)   # alive
    elif n_splits > 1:
        n_splits = 1                         # no short request in the step: the split-key kernel does not run
    prefill_tc = bool(run_prefill and tma and USE_TC_ATTENTION and head_dim == 128)
    return (tma, balanced, n_splits, short, run_decode, run_prefill, prefill_tc, _ptr(o_part), _ptr(ml_part),
            _ptr(counters), _status_word(device).data_ptr(), ctx.qo_indptr.data_ptr(), ctx.positions.data_ptr(),
            ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
            _ptr(getattr(ctx, "kv_len", None)))


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, ctx, tables, n_heads: int,
                    n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal attention of the step's tokens over their requests' cached keys.
    ``qkv``: [n, >= n_heads*head_dim] rows with the (already rotated) query heads
    first.  ``ctx`` gives qo_indptr / positions / n_entries / max_q_len, ``tables``
    the block tables of the cache group.  bfloat16 with head_dim 64/128/256 runs
    on the tensor-core kernels; everything else on the generic float32-math kernel."""
    _require_cuda(qkv, out, cache)
    assert qkv.stride(1) == 1 and out.is_contiguous() and out.dtype == qkv.dtype == cache.dtype
    lib = load_library()
    if qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256) and not FORCE_GENERIC_ATTENTION:
        # Everything that depends on the step and the layer's sizes only is worked out once per step (all layers of
        # a model ask the same question), the scratch included: the layers run one after the other on one stream.
        key = ("attention", n_heads, n_kv_heads, head_dim, id(tables), BALANCED_ATTENTION, USE_TMA_ATTENTION)
        plan = ctx.extras.get(key)
        if plan is None:
            plan = ctx.extras[key] = _attention_plan(qkv.device, ctx, tables, n_heads, n_kv_heads, head_dim)
        (tma, balanced, n_splits, short, run_decode, run_prefill, prefill_tc, o_part, ml_part, counters, status, qo, pos,
         tok_entry, kv_indptr, kv_indices, kv_len) = plan
        if prefill_tc:
            # long portions on the tcgen05 kernel; what is left for the call below are the short requests
            _check(lib.bspec_attention_prefill_tc(
                qkv.data_ptr(), qkv.stride(0), out.data_ptr(), status, cache.shape[0], cache.data_ptr(), qo, pos,
                kv_indptr, kv_indices, ctx.n_entries, qkv.shape[0], ctx.max_q_len, n_heads, n_kv_heads, head_dim,
                tables.page_size,
                float(scale), int(window), short + 1, _work_counter(qkv.device).data_ptr(), _stream()),
                "attention_prefill_tc")
            run_prefill = 0
            if not run_decode:
                return
        _check(lib.bspec_attention_bf16(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), o_part, ml_part, counters, status,
            cache.shape[0] if tma else 0, cache.data_ptr(), qo, pos, tok_entry, kv_indptr, kv_indices, ctx.n_entries,
            ctx.n_tokens, ctx.max_q_len, n_heads, n_kv_heads, head_dim, tables.page_size, float(scale), int(window),
            n_splits, short, run_decode, run_prefill, balanced, kv_len, cache.shape[0], _stream()), "attention_bf16")
        global _launches
        _launches += 1 if run_decode and run_prefill else 0
        return
    _check(lib.bspec_attention_generic(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), cache.data_ptr(), _dtype_code(qkv.dtype),
        ctx.qo_indptr.data_ptr(), ctx.positions.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
        ctx.n_entries, ctx.max_q_len, n_heads, n_kv_heads, head_dim, tables.page_size, float(scale), int(window),
        cache.shape[0], _stream()), "attention_generic")


# ---------------------------------------------------------------------------- matrix products

# Which bfloat16 products run on this package's tcgen05 kernel: "auto" (those with at most TC_GEMM_MAX_M rows),
# "all", or "none".  Measured on B200 in whole decode steps of 1B to 8B models: with up to 8 tokens the kernel (weights
# on the accumulator rows, K slices joined inside a cluster, the gate/up activation in its epilogue, weight tiles
# fetched before the wait on the kernel before) beats the vendor library by 2 to 12 %; from 16 tokens on the library
# wins, by 1 to 15 % (the join of the slices grows with the tokens), so larger steps go to the library.
TC_GEMM = "auto"
TC_GEMM_MAX_M = 8
_status = {}


def _status_word(device) -> torch.Tensor:
    if device not in _status:
        _status[device] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _status[device]


def _raise_status(dev, code: int) -> None:
    with torch.inference_mode():          # the words may have been made inside inference mode (by a step)
        _status[dev].zero_()
        for bufs in _tile_counters.values():
            for b in bufs:
                b.zero_()
        for b in _work_counters.values():
            b.zero_()
    raise KernelError(f"a kernel on {dev} gave up a bounded wait (code {code}: GEMM 1 = stage never freed, "
                      f"2 = operands never arrived, 3 = accumulator never completed; decode attention 11/13 = stage "
                      f"never freed, 12/14 = keys never arrived; prompt attention 21/22 the same, 31-41 = a role of "
                      f"the tensor-core prompt kernel).  The results of the steps "
                      f"since the last check are not valid.")


def check_status() -> None:
    """Raise if a kernel of this package gave up on a bounded wait (synchronises); in a checked build
    (``BSPEC_BOUNDS=1``) also if an index was found outside its range."""
    for dev, t in _status.items():
        code = int(t.item())
        if code:
            _raise_status(dev, code)
    check_bounds()


_BOUNDS_REPORTS = ["bspec_bounds_report_elementwise", "bspec_bounds_report_gemm_tcgen05",
                   "bspec_bounds_report_attention_generic", "bspec_bounds_report_attention_bf16"]
BOUNDS_CODES = {101: "token id (embedding)", 102: "row (gather)", 103: "block-table slot (rotary + cache append)",
                104: "page id (rotary + cache append)", 105: "block-table slot (q/k/v product's epilogue)",
                106: "page id (q/k/v product's epilogue)", 107: "page id (attention over plain loads)",
                108: "page id (bfloat16 attention over plain loads)"}


def bounds_reports() -> list:
    """Checked build only (the library built with ``BSPEC_BOUNDS=1`` in the environment): what the kernels of the
    current device recorded since the last call, as (source file, what, value, limit, block); the records are
    cleared.  Empty in an ordinary build.  Waits for the device."""
    lib = load_library()
    found = []
    for name in _BOUNDS_REPORTS:
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(c_int * 4)]
        fn.restype = c_int
        rec = (c_int * 4)()
        r = fn(ctypes.byref(rec))
        if r < 0:
            raise KernelError(f"{name} failed with CUDA error {-r}")
        if r == 1 and rec[0]:
            found.append((name[len("bspec_bounds_report_"):], BOUNDS_CODES.get(rec[0], str(rec[0])), rec[1], rec[2], rec[3]))
    return found


def bounds_build() -> bool:
    """Whether the loaded library is the checked build."""
    load_library()
    return _BOUNDS_ACTIVE


def check_bounds() -> None:
    """Raise if the checked build recorded an index outside its range (no-op in an ordinary build)."""
    if not _BOUNDS_ACTIVE:
        return
    found = bounds_reports()
    if found:
        raise KernelError("the checked build found indices outside their ranges (the accesses were skipped): " +
                          "; ".join(f"{src}: {what} {value} not in [0, {limit}) in block {block}"
                                    for src, what, value, limit, block in found))


_status_host = {}


def status_to_host_async() -> None:
    """Enqueue, on the current stream, a copy of the status word into pinned host memory: whoever synchronises
    with the stream next (to read a step's tokens or logits) calls ``raise_if_gave_up`` afterwards, so that a step
    whose kernels gave up a wait is never taken for a result, at no extra synchronisation."""
    for dev, t in _status.items():
        if dev not in _status_host:
            _status_host[dev] = torch.zeros((1,), dtype=torch.int32).pin_memory()
        _status_host[dev].copy_(t, non_blocking=True)


def raise_if_gave_up() -> None:
    """After a synchronisation that followed ``status_to_host_async``: raise if the copy shows a wait given up."""
    for dev, h in _status_host.items():
        code = int(h[0])
        if code:
            with torch.inference_mode():
                h.zero_()
            torch.cuda.synchronize(dev)
            _raise_status(dev, code)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T on the tcgen05 kernel (bfloat16 operands, float32 accumulation)."""
    lib = load_library()
    M, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    if K % 8 != 0 or M <= 0:
        raise KernelError(f"gemm_tc: sizes M={M} N={N} K={K} are not supported (K must be a multiple of 8)")
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(lib.bspec_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(out_dtype == torch.float32), 0,
                             _status_word(x.device).data_ptr(), sm_count(x.device), _stream()), "gemm_tc")
    return out


FUSE_QKV_ROPE = True       # decode-sized steps: rotary encoding and the cache append in the q/k/v product's epilogue


def linear_qkv_rope(x: torch.Tensor, wqkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool, positions: torch.Tensor,
                    tok_entry: torch.Tensor, kv_indptr: torch.Tensor, kv_indices: torch.Tensor, cache: torch.Tensor,
                    page_size: int, write_kv: bool = True) -> Optional[torch.Tensor]:
    """x [M, K] @ [Wq; Wk; Wv]^T with the rotary encoding of q and k and the write of k and v into their cache
    pages done in the product's epilogue, for bfloat16 steps of at most ``TC_GEMM_MAX_M`` tokens and heads of
    128 rotated over their whole width.  Returns [M, (Hq + 2 Hkv) * 128] whose q columns hold the rotated queries
    (its k and v columns are not written), or None when the sizes are not these: the caller then runs the product,
    ``rope_kv_append`` and so on one after the other."""
    M, K = x.shape
    N = wqkv.shape[0]
    if not (FUSE_QKV_ROPE and TC_GEMM != "none" and x.dtype == torch.bfloat16
            and cache.dtype == torch.bfloat16 and head_dim == 128 and rotary_dim == 128 and 0 < M <= TC_GEMM_MAX_M
            and K % 8 == 0 and N == (n_heads + 2 * n_kv_heads) * 128 and x.is_contiguous() and wqkv.is_contiguous()):
        return None
    _require_cuda(x, wqkv, cache, positions)
    assert inv_freq.dtype == torch.float32 and inv_freq.shape == (2, 64) and inv_freq.is_contiguous()
    assert cache.is_contiguous() and positions.dtype == torch.int32 and tok_entry.dtype == torch.int32
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _check(load_library().bspec_gemm_tc_qkv_rope(
        x.data_ptr(), wqkv.data_ptr(), out.data_ptr(), M, N, K, _status_word(x.device).data_ptr(), sm_count(x.device),
        inv_freq.data_ptr(), positions.data_ptr(), tok_entry.data_ptr(), kv_indptr.data_ptr(), kv_indices.data_ptr(),
        cache.data_ptr(), n_heads, n_kv_heads, int(page_size), int(bool(interleaved)), int(bool(write_kv)),
        cache.shape[0], _stream()), "gemm_tc_qkv_rope")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K] @ w[N, K]^T -> [M, N] in ``out_dtype`` (default: x's dtype)."""
    _require_cuda(x, w)
    out_dtype = out_dtype or x.dtype
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype, (x.shape, w.shape, x.dtype, w.dtype)
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32 and x.stride(1) == 1 and w.stride(1) == 1
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        _check(load_library().bspec_sgemm_tn(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, x.stride(0),
                                             w.stride(0), N, _stream()), "sgemm_tn")
        return out
    if (K % 8 == 0 and M > 0 and x.is_contiguous() and w.is_contiguous()
            and (TC_GEMM == "all" or (TC_GEMM == "auto" and M <= TC_GEMM_MAX_M))):
        return gemm_tc(x, w, out_dtype)
    if out_dtype == x.dtype:
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=out_dtype)


# ---------------------------------------------------------------------------- sampling

def _pick_scratch(logits: torch.Tensor):
    rows, vocab = logits.shape
    nb = load_library().bspec_pick_slices(vocab)
    part_v = torch.empty((rows * nb,), dtype=torch.float32, device=logits.device)
    part_i = torch.empty((rows * nb,), dtype=torch.int32, device=logits.device)
    return part_v, part_i


def argmax(logits: torch.Tensor) -> torch.Tensor:
    _require_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    if logits.shape[0] == 0:
        return out
    part_v, part_i = _pick_scratch(logits)
    _check(load_library().bspec_argmax(logits.data_ptr(), logits.shape[0], logits.shape[1], part_v.data_ptr(),
                                       part_i.data_ptr(), out.data_ptr(), _stream()), "argmax")
    count_launches(1)
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           stream_id: torch.Tensor, counter: torch.Tensor, seed: int,
           threshold_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row parameters on the device: temperature f32 (<= 0: greedy), top_k i32
    (<= 0: off), top_p f32 (<= 0 or >= 1: off), stream_id i64 and counter i64 (the
    random stream of the row's request and the index of the draw in it).
    ``threshold_out`` (int32 [rows]) receives each row's threshold: the ordered key
    (sign bit flipped for positive floats, all bits for negative) of the smallest
    logit that stays in the top-k / top-p set, 0 where nothing is cut."""
    _require_cuda(logits, temperature, top_k, top_p, stream_id, counter)
    rows = logits.shape[0]
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    assert temperature.dtype == torch.float32 and top_k.dtype == torch.int32 and top_p.dtype == torch.float32
    assert stream_id.dtype == torch.int64 and counter.dtype == torch.int64
    out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if rows == 0:
        return out
    part_v, part_i = _pick_scratch(logits)
    threshold = threshold_out if threshold_out is not None else torch.empty((rows,), dtype=torch.int32, device=logits.device)
    assert threshold.dtype == torch.int32 and threshold.numel() == rows and threshold.is_cuda
    _check(load_library().bspec_sample(logits.data_ptr(), rows, logits.shape[1], temperature.data_ptr(),
                                       top_k.data_ptr(), top_p.data_ptr(), stream_id.data_ptr(), counter.data_ptr(),
                                       int(seed) & 0xFFFFFFFFFFFFFFFF, threshold.data_ptr(), part_v.data_ptr(),
                                       part_i.data_ptr(), out.data_ptr(), _stream()), "sample")
    count_launches(3)
    return out
