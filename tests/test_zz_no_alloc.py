"""The decode-attention entry point for callers that cannot allocate device memory
(batchspec_b200/csrc/attention_noalloc.h): a host inside a stream capture, a
real-time loop, a process whose memory budget belongs to another allocator.  Its
scratch is a fixed array inside the library, so this test calls it the way such a
caller would: through the exported C symbol, with raw pointers, twice in a row on
different inputs (the second call meets the first call's leftovers in the shared
array), and compares each result with a float32 reference computed here with plain
torch products, and with the engine's ordinary attention entry point.  The cases
cover one split (no scratch at all), several splits, two new tokens per request,
a group of 20 query heads per key head (two row tiles, which changes how the
counters are indexed) and a window.  It also checks that sizes beyond the array
(partial results, or counters alone) are refused without a launch.

Collected last on purpose: a failure here must not hide the other tests from a
run that stops at the first failure.
"""
import ctypes
import math
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
    from batchspec_b200.kernels import ops
    ops.load_library()
    lib = ctypes.CDLL(ops.library_file())
    fn = lib.bspec_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_char_p, c_int]
    fn.restype = c_int
    return fn


def _case(seed, Hq, Hkv, hd, page, kv_lens, q_lens=None):
    g = torch.Generator(device=DEV).manual_seed(seed)
    q_lens = q_lens or [1] * len(kv_lens)
    n_entries, n = len(kv_lens), sum(q_lens)
    pages_per = [-(-L // page) for L in kv_lens]
    n_pages = sum(pages_per) + 1
    cache = (torch.randn(n_pages, 2, Hkv, page, hd, device=DEV, generator=g) * 0.7).bfloat16()
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, device=DEV, generator=g).bfloat16()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    qo = [0] + list(np.cumsum(q_lens))
    ctx = SimpleNamespace(qo_indptr=i32(qo),
                          positions=i32([L - ql + i for ql, L in zip(q_lens, kv_lens) for i in range(ql)]),
                          tok_entry=i32([e for e, ql in enumerate(q_lens) for _ in range(ql)]), n_entries=n_entries,
                          n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens), extras={"min_q_len": min(q_lens)})
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[:sum(pages_per)]
    tables = SimpleNamespace(kv_indptr=i32([0] + list(np.cumsum(pages_per))), kv_indices=perm.to(DEV, torch.int32),
                             page_size=page)
    return qkv, cache, ctx, tables


def _reference(qkv, cache, ctx, tables, Hq, Hkv, hd, scale, window, kv_lens, q_lens):
    """float32 softmax attention with plain torch products, request by request."""
    G, page = Hq // Hkv, tables.page_size
    out = torch.empty(ctx.n_tokens, Hq, hd, device=DEV)
    qo, indptr = ctx.qo_indptr.tolist(), tables.kv_indptr.tolist()
    for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):
        pages = cache[tables.kv_indices[indptr[e]:indptr[e + 1]].long()].float()         # [pages, 2, Hkv, page, hd]
        k = pages[:, 0].permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :L]
        v = pages[:, 1].permute(1, 0, 2, 3).reshape(Hkv, -1, hd)[:, :L]
        q = qkv[qo[e]:qo[e + 1], :Hq * hd].float().view(ql, Hkv, G, hd)
        s = torch.einsum("qkgd,kld->qkgl", q, k) * scale
        pos = torch.arange(L - ql, L, device=DEV)[:, None, None, None]
        key = torch.arange(L, device=DEV)[None, None, None, :]
        dead = key > pos
        if window:
            dead = dead | (key < pos - window + 1)
        p = torch.softmax(s.masked_fill(dead, float("-inf")), dim=-1)
        out[qo[e]:qo[e + 1]] = torch.einsum("qkgl,kld->qkgd", p, v).reshape(ql, Hq, hd)
    return out.view(ctx.n_tokens, Hq * hd)


CASES = [
    # Hq, Hkv, hd, page, window, two calls of (seed, kv_lens, q_lens, splits)
    (32, 8, 128, 16, 0, [(1, [700, 33, 1201, 64], None, 5), (2, [90, 1500, 257], None, 3)]),
    (8, 2, 64, 8, 0, [(3, [700, 33, 1201, 64], None, 1), (4, [90, 1500, 257], None, 4)]),           # one split: no scratch
    (8, 2, 128, 16, 0, [(5, [300, 70, 1000], [2, 1, 2], 6), (6, [64, 65], [2, 2], 2)]),             # two new tokens
    (40, 2, 64, 16, 0, [(7, [100, 1000, 3], None, 4), (8, [500, 17], None, 7)]),                    # two row tiles
    (8, 2, 128, 16, 200, [(9, [1200, 90, 700, 64], [1, 1, 2, 1], 5), (10, [450, 201], None, 2)]),   # a window
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"H{c[0]}k{c[1]}d{c[2]}w{c[4]}")
def test_no_alloc_entry_point_matches_the_reference_twice_in_a_row(lib, case):
    from batchspec_b200.kernels import ops
    Hq, Hkv, hd, page, window, calls = case
    scale = 1.0 / math.sqrt(hd)
    for call, (seed, kv_lens, q_lens, splits) in enumerate(calls):
        q_lens = q_lens or [1] * len(kv_lens)
        qkv, cache, ctx, tables = _case(seed, Hq, Hkv, hd, page, kv_lens, q_lens)
        n = ctx.n_tokens
        want = _reference(qkv, cache, ctx, tables, Hq, Hkv, hd, scale, window, kv_lens, q_lens)
        ordinary = torch.empty(n, Hq * hd, device=DEV, dtype=torch.bfloat16)
        ops.paged_attention(qkv, ordinary, cache, ctx, tables, Hq, Hkv, hd, scale, window)
        got = torch.full_like(ordinary, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        msg = ctypes.create_string_buffer(256)
        rc = lib(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), cache.data_ptr(), ctx.qo_indptr.data_ptr(),
                 ctx.positions.data_ptr(), ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(),
                 tables.kv_indices.data_ptr(), ctx.n_entries, n, ctx.max_q_len, Hq, Hkv, hd, page, scale, window, splits,
                 torch.cuda.current_stream().cuda_stream, msg, 256)
        assert rc == 0, (rc, msg.value)
        torch.cuda.synchronize()
        if call > 0:                       # after the first call's set-up nothing may be taken from the device
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=2e-2)
        torch.testing.assert_close(got.float(), ordinary.float(), rtol=3e-2, atol=2e-2)


def test_no_alloc_entry_point_refuses_what_does_not_fit(lib):
    qkv, cache, ctx, tables = _case(3, 32, 8, 128, 16, [100] * 4)
    out = torch.zeros(4, 32 * 128, device=DEV, dtype=torch.bfloat16)
    msg = ctypes.create_string_buffer(256)
    args = lambda n_tokens, q_len, splits: (
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), cache.data_ptr(), ctx.qo_indptr.data_ptr(),
        ctx.positions.data_ptr(), ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(), tables.kv_indices.data_ptr(),
        4, n_tokens, q_len, 32, 8, 128, 16, 0.1, 0, splits, torch.cuda.current_stream().cuda_stream, msg, 256)
    assert lib(*args(100000, 1, 8)) == -1 and b"scratch" in msg.value          # beyond the built-in array
    assert lib(*args(4, 50, 2)) == -2 and b"new tokens" in msg.value           # not a decode step
    # the partial results would fit, the arrival counters would not (one per request, key head and row tile)
    counters_only = (qkv.data_ptr(), qkv.stride(0), out.data_ptr(), cache.data_ptr(), ctx.qo_indptr.data_ptr(),
                     ctx.positions.data_ptr(), ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(),
                     tables.kv_indices.data_ptr(), 2100, 2100, 1, 8, 8, 64, 16, 0.1, 0, 2,
                     torch.cuda.current_stream().cuda_stream, msg, 256)
    assert 2100 * 8 * 2 * 66 <= 4 * 1024 * 1024 and 2100 * 8 > 16 * 1024
    assert lib(*counters_only) == -1 and b"counters" in msg.value
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0, "a refused call must not launch anything"
