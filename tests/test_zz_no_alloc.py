"""The decode-attention entry point for callers that cannot allocate device memory
(batchspec_b200/csrc/attention_noalloc.h): a host inside a stream capture, a
real-time loop, a process whose memory budget belongs to another allocator.  Its
scratch is a fixed array inside the library, so this test calls it the way such a
caller would: through the exported C symbol, with raw pointers, twice in a row on
different inputs (the second call meets the first call's leftovers in the shared
array), and compares each result with the engine's ordinary attention entry point.
It also checks that sizes beyond the array are refused without a launch.

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


def _case(seed, Hq, Hkv, hd, page, kv_lens):
    g = torch.Generator(device=DEV).manual_seed(seed)
    n = len(kv_lens)
    pages_per = [-(-L // page) for L in kv_lens]
    n_pages = sum(pages_per) + 1
    cache = (torch.randn(n_pages, 2, Hkv, page, hd, device=DEV, generator=g) * 0.7).bfloat16()
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, device=DEV, generator=g).bfloat16()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(qo_indptr=i32(list(range(n + 1))), positions=i32([L - 1 for L in kv_lens]),
                          tok_entry=i32(list(range(n))), n_entries=n, n_tokens=n, max_q_len=1,
                          max_kv_len=max(kv_lens), extras={"min_q_len": 1})
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[:sum(pages_per)]
    tables = SimpleNamespace(kv_indptr=i32([0] + list(np.cumsum(pages_per))), kv_indices=perm.to(DEV, torch.int32),
                             page_size=page)
    return qkv, cache, ctx, tables


@pytest.mark.parametrize("shape", [(32, 8, 128, 16), (8, 2, 64, 8)])
def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row(lib, shape):
    from batchspec_b200.kernels import ops
    Hq, Hkv, hd, page = shape
    for call, (seed, kv_lens, splits) in enumerate([(1, [700, 33, 1201, 64], 5), (2, [90, 1500, 257], 3)]):
        qkv, cache, ctx, tables = _case(seed, Hq, Hkv, hd, page, kv_lens)
        n = ctx.n_tokens
        want = torch.empty(n, Hq * hd, device=DEV, dtype=torch.bfloat16)
        ops.paged_attention(qkv, want, cache, ctx, tables, Hq, Hkv, hd, 1.0 / math.sqrt(hd), 0)
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        msg = ctypes.create_string_buffer(256)
        rc = lib(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), cache.data_ptr(), ctx.qo_indptr.data_ptr(),
                 ctx.positions.data_ptr(), ctx.tok_entry.data_ptr(), tables.kv_indptr.data_ptr(),
                 tables.kv_indices.data_ptr(), n, n, 1, Hq, Hkv, hd, page, 1.0 / math.sqrt(hd), 0, splits,
                 torch.cuda.current_stream().cuda_stream, msg, 256)
        assert rc == 0, (rc, msg.value)
        torch.cuda.synchronize()
        if call > 0:                       # after the first call's set-up nothing may be taken from the device
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=2e-2)


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
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0, "a refused call must not launch anything"
