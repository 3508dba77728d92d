"""Each CUDA kernel alone against a plain float32 PyTorch reference of the same
operation, at sizes other than the engine's tiny models: widths and vocabularies
that are no power of two, head sizes from 16 to 256, odd group sizes, page sizes
from 1 up, ragged batches."""
import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from batchspec_b200.kernels import ops
    ops.load_library()
    return ops


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,d,vocab", [(1, 48, 7), (37, 1000, 333), (5, 4096, 50)])
def test_embed(ops, dtype, n, d, vocab):
    g = torch.Generator(device=DEV).manual_seed(0)
    table = torch.randn(vocab, d, device=DEV, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (n,), device=DEV, generator=g, dtype=torch.int32)
    out = torch.empty(n, d, device=DEV)
    ops.embed(ids, table, out, 1.5)
    assert torch.equal(out, table[ids.long()].float() * 1.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wdtype", [torch.float32, None])
@pytest.mark.parametrize("n,d,eps", [(3, 96, 1e-6), (17, 1000, 1e-5), (2, 4096, 1e-2), (1, 6144, 1e-5),
                                     (600, 4096, 1e-5), (513, 1000, 1e-5), (520, 8192, 1e-5)])
def test_add_rmsnorm(ops, dtype, wdtype, n, d, eps):
    g = torch.Generator(device=DEV).manual_seed(1)
    resid = torch.randn(n, d, device=DEV, generator=g) * 3
    delta = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)).to(wdtype or dtype)
    want_resid = resid + delta.float()
    normed = want_resid * torch.rsqrt((want_resid * want_resid).mean(-1, keepdim=True) + eps)
    want = (normed.to(dtype).float() * w.float()).to(dtype)           # cast, then scale (reference order)
    out = torch.empty(n, d, device=DEV, dtype=dtype)
    r = resid.clone()
    ops.add_rmsnorm(r, delta, w, eps, out)
    assert torch.equal(r, want_resid), "the residual sum is exact float32"
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))
    out2 = torch.empty_like(out)
    r2 = want_resid.clone()
    ops.add_rmsnorm(r2, None, w, eps, out2)                            # without a pending branch
    assert torch.equal(out, out2) and torch.equal(r2, want_resid)


def test_gather_rows_add(ops):
    g = torch.Generator(device=DEV).manual_seed(2)
    resid = torch.randn(9, 200, device=DEV, generator=g)
    pend = torch.randn(9, 200, device=DEV, generator=g).bfloat16()
    rows = torch.tensor([8, 0, 3, 3], device=DEV, dtype=torch.int32)
    out = torch.empty(4, 200, device=DEV)
    ops.gather_rows_add(resid, pend, rows, out)
    assert torch.equal(out, resid[rows.long()] + pend[rows.long()].float())
    ops.gather_rows_add(resid, None, rows, out)
    assert torch.equal(out, resid[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,inter", [(1, 7), (13, 176), (4, 14336)])
def test_silu_mul(ops, dtype, n, inter):
    g = torch.Generator(device=DEV).manual_seed(3)
    u = (torch.randn(n, 2 * inter, device=DEV, generator=g) * 4).to(dtype)
    out = torch.empty(n, inter, device=DEV, dtype=dtype)
    ops.silu_mul(u, out)
    gate, up = u[:, :inter].float(), u[:, inter:].float()
    torch.testing.assert_close(out.float(), (gate * torch.sigmoid(gate) * up).to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 5, 3), (7, 130, 96), (64, 64, 16), (65, 1000, 257), (300, 33, 1024)])
def test_sgemm_is_true_float32(ops, M, N, K):
    g = torch.Generator(device=DEV).manual_seed(4)
    a = torch.randn(M, K, device=DEV, generator=g)
    w = torch.randn(N, K, device=DEV, generator=g)
    got = ops.linear(a, w)
    want = (a.double() @ w.double().T)
    err = (got.double() - want).abs().max().item()
    assert err <= 1e-6 * K ** 0.5 * 16, err                       # float32 accumulation error, far below tf32's 1e-3
    # a row's result does not depend on the other rows of the batch
    assert torch.equal(got[:1], ops.linear(a[:1].contiguous(), w))


def _rope_reference(x, pos, inv_freq, rot, interleaved):
    """float64 angle from the float32 frequencies given, float32 result."""
    ang = pos.double()[:, None] * inv_freq.double()[None, :]
    c, s = torch.cos(ang)[:, None, :].float(), torch.sin(ang)[:, None, :].float()
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, a * s + b * c
    else:
        a, b = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2], out[..., rot // 2:rot] = a * c - b * s, a * s + b * c
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lens", [[3, 1, 9], [70, 1, 200], [600]])           # few tokens; many (16-byte path in bfloat16)
@pytest.mark.parametrize("Hq,Hkv,hd,rot,inter,ps", [(4, 2, 16, 16, False, 4), (3, 1, 32, 32, True, 1),
                                                     (6, 3, 48, 24, False, 5), (32, 8, 128, 128, False, 16),
                                                     (5, 1, 80, 80, False, 8)])
def test_rope_and_cache_append(ops, dtype, Hq, Hkv, hd, rot, inter, ps, lens):
    g = torch.Generator(device=DEV).manual_seed(5)
    before = [0, 6, 11][:len(lens)]                              # new tokens per request after tokens already cached
    n = sum(lens)
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, device=DEV, generator=g).to(dtype)
    inv_freq = (10000.0 ** (-torch.arange(0, rot // 2, device=DEV).float() * 2 / rot))
    table = ops.rope_frequency_table(inv_freq, DEV)
    pos = torch.cat([torch.arange(b, b + l) for l, b in zip(lens, before)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((l,), i) for i, l in enumerate(lens)]).to(DEV, torch.int32)
    pages_per = [-(-(b + l) // ps) for l, b in zip(lens, before)]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6))[:sum(pages_per)]
    indptr = torch.tensor([0] + list(np.cumsum(pages_per)), dtype=torch.int32, device=DEV)
    indices = perm.to(DEV, torch.int32)
    cache = torch.full((n_pages, 2, Hkv, ps, hd), 7.0, device=DEV, dtype=dtype)
    ref_q = _rope_reference(qkv[:, :Hq * hd].float().view(n, Hq, hd), pos, inv_freq, rot, inter).to(dtype)
    ref_k = _rope_reference(qkv[:, Hq * hd:(Hq + Hkv) * hd].float().view(n, Hkv, hd), pos, inv_freq, rot, inter).to(dtype)
    v = qkv[:, (Hq + Hkv) * hd:].view(n, Hkv, hd).clone()
    work = qkv.clone()
    ops.rope_kv_append(work, Hq, Hkv, hd, table, rot, inter, pos, ent, indptr, indices, cache, ps)
    torch.testing.assert_close(work[:, :Hq * hd].float().view(n, Hq, hd), ref_q.float(), **tol(dtype))
    want = torch.full_like(cache, 7.0)
    for t in range(n):
        e, p = int(ent[t]), int(pos[t])
        page = int(indices[int(indptr[e]) + p // ps])
        want[page, 0, :, p % ps, :] = ref_k[t]
        want[page, 1, :, p % ps, :] = v[t]
    torch.testing.assert_close(cache.float(), want.float(), **tol(dtype))
    assert torch.equal(cache[:, 1], want[:, 1]), "values are copied bit for bit"
    untouched = torch.ones(n_pages, dtype=torch.bool)
    untouched[perm] = False
    assert bool((cache[untouched.to(DEV)] == 7.0).all()), "pages of no request were written"
    # read-only run (a layer that shares another layer's cache): q rotated, cache untouched
    cache2 = torch.full_like(cache, 7.0)
    work2 = qkv.clone()
    ops.rope_kv_append(work2, Hq, Hkv, hd, table, rot, inter, pos, ent, indptr, indices, cache2, ps, write_kv=False)
    assert torch.equal(work2[:, :Hq * hd], work[:, :Hq * hd]) and bool((cache2 == 7.0).all())
    # the stand-alone rotation agrees with the fused one
    alone = qkv.clone()
    ops.rope_inplace(alone[:, :Hq * hd].view(n, Hq, hd), pos, table, rot, inter)
    assert torch.equal(alone[:, :Hq * hd], work[:, :Hq * hd])


@pytest.mark.parametrize("inter", [False, True])
@pytest.mark.parametrize("M,Hq,Hkv,K", [(1, 32, 8, 4096), (8, 32, 8, 4096), (3, 5, 1, 512), (7, 4, 2, 328), (8, 24, 8, 3072)])
def test_qkv_projection_with_rope_and_cache_append_in_its_epilogue(ops, M, Hq, Hkv, K, inter):
    """The fused kernel of decode-sized steps against float64 arithmetic: rotated q in the output, rotated k and
    plain v in the right rows of the right pages, nothing else in the cache touched; one K slice and several."""
    hd, ps = 128, 16
    g = torch.Generator(device=DEV).manual_seed(M + Hq)
    N = (Hq + 2 * Hkv) * hd
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).bfloat16()
    import plain_llama as P
    freqs = P.rope_frequencies(dict(head_dim=hd, rope_theta=500000.0, hidden_size=Hq * hd, num_attention_heads=Hq,
                                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                                      high_freq_factor=4.0, original_max_position_embeddings=8192)))
    table = ops.rope_frequency_table(freqs, DEV)
    kv_before = [5, 130, 31, 64, 1000, 15, 16, 99999][:M]          # one new token per request, at these positions
    positions = torch.tensor(kv_before, dtype=torch.int32, device=DEV)
    ent = torch.arange(M, dtype=torch.int32, device=DEV)
    pages_per = [-(-(b + 1) // ps) for b in kv_before]
    # a table as long as each request, whose last entry is the request's own page (the only one written)
    indptr = torch.tensor([0] + list(np.cumsum(pages_per)), dtype=torch.int32, device=DEV)
    indices = torch.zeros(sum(pages_per), dtype=torch.int32)
    own = torch.randperm(M + 2, generator=torch.Generator().manual_seed(9))[:M] + 1
    for e in range(M):
        indices[int(indptr[e + 1]) - 1] = own[e]
    indices = indices.to(DEV)
    cache = torch.full((M + 3, 2, Hkv, ps, hd), 7.0, device=DEV, dtype=torch.bfloat16)
    got = ops.linear_qkv_rope(x, w, Hq, Hkv, hd, table, hd, inter, positions, ent, indptr, indices, cache, ps)
    assert got is not None, "these sizes are the fused kernel's"
    torch.cuda.synchronize()
    ops.check_status()
    qkv = (x.double() @ w.double().T).cpu()
    ang = positions.cpu().double()[:, None] * freqs[None, :]
    c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rotate(t):
        out = torch.empty_like(t)
        if inter:
            a, b = t[..., 0::2], t[..., 1::2]
            out[..., 0::2], out[..., 1::2] = a * c - b * s_, a * s_ + b * c
        else:
            a, b = t[..., :hd // 2], t[..., hd // 2:]
            out[..., :hd // 2], out[..., hd // 2:] = a * c - b * s_, a * s_ + b * c
        return out

    want_q = rotate(qkv[:, :Hq * hd].view(M, Hq, hd))
    want_k = rotate(qkv[:, Hq * hd:(Hq + Hkv) * hd].view(M, Hkv, hd))
    want_v = qkv[:, (Hq + Hkv) * hd:].view(M, Hkv, hd)
    tol = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got[:, :Hq * hd].view(M, Hq, hd).double().cpu(), want_q, **tol)
    touched = torch.zeros(M + 3, ps, dtype=torch.bool)
    for e in range(M):
        page, row = int(own[e]), kv_before[e] % ps
        touched[page, row] = True
        torch.testing.assert_close(cache[page, 0, :, row].double().cpu(), want_k[e], **tol)
        torch.testing.assert_close(cache[page, 1, :, row].double().cpu(), want_v[e], **tol)
    untouched = cache.cpu().permute(0, 3, 1, 2, 4)[~touched]
    assert bool((untouched == 7.0).all()), "only the new tokens' rows are written"
    # a run that only reads the cache (a layer that shares another layer's) writes nothing
    cache2 = torch.full_like(cache, 7.0)
    got2 = ops.linear_qkv_rope(x, w, Hq, Hkv, hd, table, hd, inter, positions, ent, indptr, indices, cache2, ps,
                               write_kv=False)
    assert torch.equal(got2[:, :Hq * hd], got[:, :Hq * hd]) and bool((cache2 == 7.0).all())
    # and it agrees with the three kernels it replaces
    plain = ops.linear(x, w)
    cache3 = torch.full_like(cache, 7.0)
    ops.rope_kv_append(plain, Hq, Hkv, hd, table, hd, inter, positions, ent, indptr, indices, cache3, ps)
    torch.testing.assert_close(got[:, :Hq * hd].float(), plain[:, :Hq * hd].float(), **tol)
    torch.testing.assert_close(cache.float(), cache3.float(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [False, True])
@pytest.mark.parametrize("n", [9, 80])                 # the per-head kernel; the 16-byte bfloat16 kernel (n >= 64)
def test_rope_at_large_positions(ops, dtype, inter, n):
    """Positions up to 131,071 with the Llama-3 base and the llama3 rule: the angle is formed in float64 on the
    device, so a float32 run stays within its own tolerance there (a float32 product position * frequency would
    be off by up to 8e-3 rad).  Every rotary pair of q holds (1, 0): the output shows cos and sin of each angle."""
    Hq, Hkv, hd, ps = 4, 2, 128, 16
    import plain_llama as P
    freqs = P.rope_frequencies(dict(head_dim=hd, rope_theta=500000.0, hidden_size=Hq * hd, num_attention_heads=Hq,
                                    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                                                      high_freq_factor=4.0, original_max_position_embeddings=8192)))
    table = ops.rope_frequency_table(freqs, DEV)
    marks = [0, 1, 8191, 8192, 32767, 32768, 131070, 131069]      # 131,071 itself only once, as the last token
    positions = torch.tensor((marks * (n // len(marks) + 1))[:n - 1] + [131071], dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, generator=g, dtype=torch.float64)
    q = qkv[:, :Hq * hd].view(n, Hq, hd)
    q[:, 0] = 0
    if inter:
        q[:, 0, 0::2] = 1.0
    else:
        q[:, 0, :hd // 2] = 1.0
    qkv = qkv.to(dtype)
    ang = positions.double()[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def rotate(x):
        x = x.double()
        out = torch.empty_like(x)
        if inter:
            a, b = x[..., 0::2], x[..., 1::2]
            out[..., 0::2], out[..., 1::2] = a * c - b * s, a * s + b * c
        else:
            a, b = x[..., :hd // 2], x[..., hd // 2:]
            out[..., :hd // 2], out[..., hd // 2:] = a * c - b * s, a * s + b * c
        return out

    want_q = rotate(qkv[:, :Hq * hd].view(n, Hq, hd))
    want_k = rotate(qkv[:, Hq * hd:(Hq + Hkv) * hd].view(n, Hkv, hd))
    work = qkv.to(DEV)
    pos = positions.to(DEV)
    ent = torch.zeros(n, dtype=torch.int32, device=DEV)
    # one request whose table gives every page that these positions touch a real page of its own
    n_table = 131072 // ps
    touched = sorted(set((positions // ps).tolist()))
    indices = torch.zeros(n_table, dtype=torch.int32)
    indices[touched] = torch.arange(1, len(touched) + 1, dtype=torch.int32)
    indices = indices.to(DEV)
    indptr = torch.tensor([0, n_table], dtype=torch.int32, device=DEV)
    cache = torch.zeros(len(touched) + 1, 2, Hkv, ps, hd, device=DEV, dtype=dtype)
    ops.rope_kv_append(work, Hq, Hkv, hd, table, hd, inter, pos, ent, indptr, indices, cache, ps)
    alone = qkv.to(DEV)
    ops.rope_inplace(alone[:, :Hq * hd].view(n, Hq, hd), pos, table, hd, inter)
    got_q = work[:, :Hq * hd].view(n, Hq, hd).double().cpu()
    assert torch.equal(alone[:, :Hq * hd], work[:, :Hq * hd])
    # float32: the reduced angle is rounded to float32 (2e-7 rad) and sine / cosine are float32
    tol = 1e-6 if dtype == torch.float32 else 2.0 ** -8
    scale = qkv.abs().max().item()
    assert (got_q[:, 0] - want_q[:, 0]).abs().max() <= tol, "the pairs that hold (1, 0) show the angle itself"
    assert (got_q - want_q).abs().max() <= tol * scale
    last = n - 1                                            # position 131,071: row 15 of the last touched page
    got_k = cache[len(touched), 0, :, 15].double().cpu()
    assert (got_k - want_k[last]).abs().max() <= tol * scale


def _attention_case(ops, dtype, Hq, Hkv, hd, ps, q_lens, kv_lens, window=0, spike=None, seed=0, force_generic=False,
                    splits=None, balanced=True, give_kv_len=False):
    """Random q/k/v, pages in scrambled order; returns (got, want)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    n_entries, G = len(q_lens), Hq // Hkv
    n = sum(q_lens)
    q = torch.randn(n, Hq * hd, device=DEV, generator=g)
    ks = [torch.randn(L, Hkv, hd, device=DEV, generator=g) for L in kv_lens]
    vs = [torch.randn(L, Hkv, hd, device=DEV, generator=g) for L in kv_lens]
    if spike is not None:                   # one far key that must dominate one query's softmax
        e, key, head = spike
        t = sum(q_lens[:e]) + q_lens[e] - 1
        q[t].view(Hq, hd)[head] = 0
        q[t].view(Hq, hd)[head, 0] = 40.0
        for kk in ks[e]:
            kk[:, 0] = kk[:, 0].clamp(-1, 1)
        ks[e][key, head // G, 0] = 30.0
    q, ks, vs = q.to(dtype), [k.to(dtype) for k in ks], [v.to(dtype) for v in vs]
    pages_per = [-(-L // ps) for L in kv_lens]
    n_pages = sum(pages_per) + 3                                       # the last one is never a request's page
    perm = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(seed + 1))[:sum(pages_per)]
    cache = torch.randn(n_pages, 2, Hkv, ps, hd, device=DEV, generator=g).to(dtype)      # garbage where nothing lives
    indptr = [0] + list(np.cumsum(pages_per))
    for e, L in enumerate(kv_lens):
        for p in range(L):
            page = int(perm[indptr[e] + p // ps])
            cache[page, 0, :, p % ps] = ks[e][p]
            cache[page, 1, :, p % ps] = vs[e][p]
    if window:
        # Pages that lie wholly before the oldest key any query of the step reads are what the cache manager has
        # given back by now.  Their table entries point at a page of huge (finite) numbers here: a kernel that
        # reads one gets a wrong result, not a wild address.
        poison = n_pages - 1
        cache[poison] = 3.0e4
        perm = perm.clone()
        for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):
            dead = max(0, (L - ql) - window + 1) // ps
            perm[indptr[e]:indptr[e] + dead] = poison
    qo = [0] + list(np.cumsum(q_lens))
    pos = torch.cat([torch.arange(L - ql, L) for ql, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((ql,), i) for i, ql in enumerate(q_lens)]).to(DEV, torch.int32)
    ctx = SimpleNamespace(qo_indptr=torch.tensor(qo, dtype=torch.int32, device=DEV), positions=pos, tok_entry=ent,
                          n_entries=n_entries, n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens),
                          extras={"min_q_len": min(q_lens), "attn_splits": splits})
    if give_kv_len:
        ctx.kv_len = torch.tensor(kv_lens, dtype=torch.int32, device=DEV)
    tables = SimpleNamespace(kv_indptr=torch.tensor(indptr, dtype=torch.int32, device=DEV),
                             kv_indices=perm.to(DEV, torch.int32), page_size=ps)
    out = torch.full((n, Hq * hd), float("nan"), device=DEV, dtype=dtype)
    scale = 1.0 / math.sqrt(hd)
    ops.FORCE_GENERIC_ATTENTION = force_generic
    was = ops.BALANCED_ATTENTION
    ops.BALANCED_ATTENTION = balanced
    try:
        ops.paged_attention(q, out, cache, ctx, tables, Hq, Hkv, hd, scale, window)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ops.FORCE_GENERIC_ATTENTION = False
        ops.BALANCED_ATTENTION = was
    want = torch.empty(n, Hq, hd, device=DEV)
    for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):
        qe = q[qo[e]:qo[e + 1]].float().view(ql, Hq, hd)
        k, v = ks[e].float(), vs[e].float()
        for i in range(ql):
            p = L - ql + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(Hq):
                s = (k[lo:p + 1, h // G] @ qe[i, h]) * scale
                want[qo[e] + i, h] = torch.softmax(s, 0) @ v[lo:p + 1, h // G]
    return out.float().view(n, Hq, hd), want


ATT_SHAPES = [
    # Hq, Hkv, hd, page, q_lens, kv_lens
    (4, 2, 16, 4, [5, 1, 2], [5, 9, 30]),
    (3, 1, 32, 1, [1, 1, 7], [40, 1, 7]),
    (6, 2, 48, 5, [3, 11], [17, 11]),
    (8, 2, 64, 16, [1, 1, 1, 1], [300, 17, 64, 129]),
    (8, 2, 64, 8, [70, 2, 1], [200, 5, 333]),
    (32, 8, 128, 16, [1, 1, 1], [700, 2049, 33]),
    (12, 4, 128, 16, [130, 1, 3, 64], [130, 555, 40, 600]),
    (5, 5, 128, 32, [9, 200], [77, 200]),
    (4, 1, 256, 16, [1, 40], [150, 90]),
    (40, 2, 64, 16, [1, 2], [100, 65]),                # 20 query heads per kv head: more than one 16-row tile
    (32, 8, 128, 16, [300], [300]),                    # head_dim 128, long portions: the tcgen05 kernel
    (32, 8, 128, 16, [128, 257, 1], [1000, 257, 90]),
    (8, 8, 128, 64, [100], [700]),
    (16, 2, 128, 8, [33, 500], [33, 777]),
    (6, 2, 128, 32, [129], [385]),                     # 3 query heads per kv head: rows do not align with tokens
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATT_SHAPES, ids=lambda s: f"H{s[0]}k{s[1]}d{s[2]}p{s[3]}")
def test_paged_attention(ops, dtype, shape):
    Hq, Hkv, hd, ps, q_lens, kv_lens = shape
    got, want = _attention_case(ops, dtype, Hq, Hkv, hd, ps, q_lens, kv_lens, seed=len(q_lens))
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else
                                             dict(rtol=3e-2, atol=2e-2)))


@pytest.mark.parametrize("splits", [1, 3, 8])
def test_split_keys_agree_with_one_pass(ops, splits):
    a, want = _attention_case(ops, torch.bfloat16, 8, 2, 128, 16, [1, 1, 2], [1000, 70, 513], splits=splits, seed=7)
    torch.testing.assert_close(a, want, rtol=3e-2, atol=2e-2)
    b, _ = _attention_case(ops, torch.bfloat16, 8, 2, 128, 16, [1, 1, 2], [1000, 70, 513], force_generic=True, seed=7)
    torch.testing.assert_close(a, b, rtol=3e-2, atol=2e-2)


@pytest.mark.parametrize("Hq,Hkv,q_lens,kv_lens", [(32, 8, [257, 1024], [8192 + 257, 30000]),
                                                   (32, 8, [1024, 257], [8192, 30000 + 257]), (32, 8, [4096], [30000]),
                                                   # 3 query heads per kv head: rows do not align with tokens, so
                                                   # the softmax threads fetch Q themselves; 168 items on 148 CTAs,
                                                   # a third of them naming no work (the shorter request)
                                                   (6, 2, [3500, 2200], [3700, 9000]),
                                                   (8, 8, [1500, 2500], [6000, 2500])])
def test_prompt_portions_deep_inside_a_long_context(ops, Hq, Hkv, q_lens, kv_lens):
    """Portions of a prompt at cached lengths of 8,192 and 30,000 tokens on the tensor-core prompt kernel
    (head_dim 128, page 16): hundreds of key tiles per query tile, several items per persistent CTA drawn
    heaviest first, pages looked up far into a scrambled table.  Queries are scaled up so that the softmax is peaked (with unit-variance
    scores over 30,000 keys every output would be near zero and any fault would hide inside the tolerance); one
    query per request also has a single far key that must win.  Reference: float32 torch products on the GPU.
    A second launch gives the same bits, whichever CTA draws which item."""
    hd, ps = 128, 16
    G = Hq // Hkv
    g = torch.Generator(device=DEV).manual_seed(11)
    n, scale = sum(q_lens), 1.0 / math.sqrt(hd)
    q = (torch.randn(n, Hq * hd, device=DEV, generator=g) * 5.0)
    ks = [torch.randn(L, Hkv, hd, device=DEV, generator=g) for L in kv_lens]
    vs = [torch.randn(L, Hkv, hd, device=DEV, generator=g) for L in kv_lens]
    qo = [0] + list(np.cumsum(q_lens))
    far = []
    for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):          # the last query's head 5 looks at key 3 alone
        t = qo[e + 1] - 1
        q[t].view(Hq, hd)[5] = 0
        q[t].view(Hq, hd)[5, 0] = 60.0
        ks[e][:, 5 // G, 0].clamp_(-1, 1)
        ks[e][3, 5 // G, 0] = 30.0
        far.append((t, e, 5, 3))
        # and head 2 at a late key: the row's scale, settled on the first tiles, is off by a factor of 2^200 when
        # that key's tile comes (the probabilities formed with the old scale overflow and the tile is done again)
        q[t].view(Hq, hd)[2] = 0
        q[t].view(Hq, hd)[2, 1] = 60.0
        ks[e][:, 2 // G, 1].clamp_(-1, 1)
        ks[e][L - 40, 2 // G, 1] = 30.0
        far.append((t, e, 2, L - 40))
    q, ks, vs = q.bfloat16(), [k.bfloat16() for k in ks], [v.bfloat16() for v in vs]
    pages_per = [-(-L // ps) for L in kv_lens]
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(12))[:sum(pages_per)]
    cache = torch.randn(n_pages, 2, Hkv, ps, hd, device=DEV, generator=g).bfloat16()
    indptr = [0] + list(np.cumsum(pages_per))
    for e, L in enumerate(kv_lens):
        pad = pages_per[e] * ps - L
        for which, src in ((0, ks[e]), (1, vs[e])):
            full = torch.cat([src, cache[0, which, :, :pad].permute(1, 0, 2)]) if pad else src
            cache[perm[indptr[e]:indptr[e + 1]].to(DEV), which] = full.view(pages_per[e], ps, Hkv, hd).permute(0, 2, 1, 3)
    pos = torch.cat([torch.arange(L - ql, L) for ql, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((ql,), i) for i, ql in enumerate(q_lens)]).to(DEV, torch.int32)
    ctx = SimpleNamespace(qo_indptr=torch.tensor(qo, dtype=torch.int32, device=DEV), positions=pos, tok_entry=ent,
                          n_entries=len(q_lens), n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens),
                          extras={"min_q_len": min(q_lens)})
    tables = SimpleNamespace(kv_indptr=torch.tensor(indptr, dtype=torch.int32, device=DEV),
                             kv_indices=perm.to(DEV, torch.int32), page_size=ps)
    out = torch.full((n, Hq * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    before = ops.launch_count()
    ops.paged_attention(q, out, cache, ctx, tables, Hq, Hkv, hd, scale, 0)
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_count() - before == 1, "only the tensor-core prompt kernel runs for these portions"
    assert not torch.isnan(out.float()).any()
    again = torch.full_like(out, float("nan"))
    ops.paged_attention(q, again, cache, ctx, tables, Hq, Hkv, hd, scale, 0)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(out, again)
    for e, (ql, L) in enumerate(zip(q_lens, kv_lens)):
        k, v = ks[e].float().permute(1, 0, 2), vs[e].float().permute(1, 0, 2)               # [Hkv, L, hd]
        key = torch.arange(L, device=DEV)[None, None, :]
        for b in range(0, ql, 256):                                                        # 256 queries at a time
            rows = slice(qo[e] + b, qo[e] + min(ql, b + 256))
            qq = q[rows].float().view(-1, Hkv, G, hd)
            sc = torch.einsum("qkgd,kld->kgql", qq, k) * scale
            p_ = pos[rows].long()[None, None, :, None]
            pr = torch.softmax(sc.masked_fill(key[None] > p_, float("-inf")), dim=-1)
            want = torch.einsum("kgql,kld->qkgd", pr, v).reshape(-1, Hq * hd)
            torch.testing.assert_close(out[rows].float(), want, rtol=3e-2, atol=2e-2)
    for t, e, head, key in far:
        torch.testing.assert_close(out[t].float().view(Hq, hd)[head], vs[e][key, head // G].float(), rtol=3e-2, atol=2e-2)


RAGGED = [
    # Hq, Hkv, hd, page, q_lens, kv_lens, window: decode-sized requests of very different lengths
    (8, 2, 128, 16, [1] * 9, [3000, 1, 64, 65, 700, 2, 1500, 129, 4000], 0),
    (32, 8, 128, 16, [1] * 40, [17 * i + 1 for i in range(40)], 0),           # more row tiles than CTAs' shares
    (6, 2, 64, 8, [2, 1, 2, 1, 1], [900, 5, 70, 2000, 333], 0),               # 3 heads per kv head, two new tokens
    (40, 2, 64, 16, [1, 1, 1], [100, 1000, 3], 0),                            # 20 heads per kv head: two row tiles
    (4, 1, 256, 32, [1, 1], [2500, 40], 0),
    (8, 2, 128, 16, [1, 1, 3, 1], [1200, 90, 700, 64], 200),                  # a window that leaves out early pages
    (8, 2, 128, 64, [1] * 3, [70000, 10, 5000], 0),                           # one request far longer than the others
]


@pytest.mark.parametrize("give_kv_len", [False, True])
@pytest.mark.parametrize("shape", RAGGED, ids=lambda s: f"H{s[0]}k{s[1]}d{s[2]}n{len(s[4])}w{s[6]}")
def test_equal_shares_of_ragged_requests(ops, shape, give_kv_len):
    """The decode kernel that gives every CTA the same number of key tiles, against the reference and against the
    kernel that cuts every request by itself."""
    Hq, Hkv, hd, ps, q_lens, kv_lens, window = shape
    got, want = _attention_case(ops, torch.bfloat16, Hq, Hkv, hd, ps, q_lens, kv_lens, window=window, seed=5,
                                give_kv_len=give_kv_len)
    assert not torch.isnan(got).any()
    torch.testing.assert_close(got, want, rtol=3e-2, atol=2e-2)
    other, _ = _attention_case(ops, torch.bfloat16, Hq, Hkv, hd, ps, q_lens, kv_lens, window=window, seed=5,
                               balanced=False)
    torch.testing.assert_close(got, other, rtol=2e-2, atol=1e-2)
    again, _ = _attention_case(ops, torch.bfloat16, Hq, Hkv, hd, ps, q_lens, kv_lens, window=window, seed=5,
                               give_kv_len=give_kv_len)
    assert torch.equal(got, again), "the same launch gives the same bits"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,q_lens,kv_lens,window", [(64, [1, 20, 3], [100, 60, 35], 17), (32, [4, 1], [50, 9], 8),
                                                      (128, [1, 90], [400, 300], 64)])
def test_window(ops, dtype, hd, q_lens, kv_lens, window):
    got, want = _attention_case(ops, dtype, 4, 2, hd, 8, q_lens, kv_lens, window=window, seed=3)
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else
                                             dict(rtol=3e-2, atol=2e-2)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key", [0, 15, 16, 511, 512, 1023, 1500])
def test_one_far_key_among_hundreds_is_found(ops, dtype, key):
    """One key, scaled so that its score stands out, decides the output: a kernel
    that skips or misplaces a page, a tile edge or a split shows here."""
    got, want = _attention_case(ops, dtype, 8, 2, 128, 16, [1, 1], [64, 1501], spike=(1, key, 5), seed=11)
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else
                                             dict(rtol=3e-2, atol=3e-2)))


def test_argmax_and_ties(ops):
    g = torch.Generator(device=DEV).manual_seed(8)
    logits = torch.randn(5, 128256, device=DEV, generator=g)
    assert torch.equal(ops.argmax(logits).long(), torch.argmax(logits, -1))
    tie = torch.zeros(2, 1000, device=DEV)
    tie[0, [400, 17, 999]] = 3.0
    tie[1, 999] = 1.0
    assert ops.argmax(tie).tolist() == [17, 999]


def _draw(ops, logits_row, n, T, top_k, top_p, seed=123, stream=5):
    logits = logits_row.to(DEV).float().repeat(n, 1).contiguous()
    f = lambda v, dt: torch.full((n,), v, device=DEV, dtype=dt)
    return ops.sample(logits, f(T, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
                      f(stream, torch.int64), torch.arange(n, device=DEV, dtype=torch.int64), seed).cpu()


def test_sampling_follows_the_softmax(ops):
    import plain_llama as P
    g = torch.Generator().manual_seed(9)
    row = torch.randn(50, generator=g) * 2
    n = 40000
    for T, k, p in [(0.8, -1, 0.0), (1.3, 7, 0.0), (0.8, -1, 0.6), (1.0, 12, 0.9)]:
        draws = _draw(ops, row, n, T, k, p)
        want = P.top_k_top_p_filter(P.softmax_temperature(row, T), k, p).numpy()
        counts = np.bincount(draws.numpy(), minlength=50)
        assert counts[want == 0].sum() == 0, "a token outside the top-k / top-p set was drawn"
        live = want > 0
        chi2 = (((counts[live] - n * want[live]) ** 2) / (n * want[live])).sum()
        assert chi2 < 3 * live.sum() + 30, (T, k, p, chi2)
    assert _draw(ops, row, 8, 0.0, -1, 0.0).tolist() == [int(row.argmax())] * 8


def test_sampling_depends_on_stream_and_counter_only(ops):
    g = torch.Generator().manual_seed(10)
    row = torch.randn(1000, generator=g)
    a = _draw(ops, row, 64, 1.0, -1, 0.0, seed=1, stream=3)
    assert torch.equal(a, _draw(ops, row, 64, 1.0, -1, 0.0, seed=1, stream=3))
    assert torch.equal(a[:5], _draw(ops, row, 5, 1.0, -1, 0.0, seed=1, stream=3)), "independent of the batch"
    assert not torch.equal(a, _draw(ops, row, 64, 1.0, -1, 0.0, seed=1, stream=4))
    assert not torch.equal(a, _draw(ops, row, 64, 1.0, -1, 0.0, seed=2, stream=3))
    assert len(set(a.tolist())) > 20


def _threshold_values(ops, logits, T, k, p):
    """The smallest logit each row keeps, read back from the sampling kernels' threshold word."""
    n = logits.shape[0]
    f = lambda v, dt: torch.full((n,), v, device=DEV, dtype=dt)
    th = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, f(T, torch.float32), f(k, torch.int32), f(p, torch.float32), f(1, torch.int64),
               torch.arange(n, device=DEV, dtype=torch.int64), 7, threshold_out=th)
    key = th.cpu().numpy().view(np.uint32)
    bits = np.where(key & 0x80000000, key & 0x7FFFFFFF, ~key).astype(np.uint32)
    return bits.view(np.float32)


@pytest.mark.parametrize("vocab", [128256, 50257, 1000])
def test_sampling_thresholds_at_large_vocabularies(ops, vocab):
    """The cut of top-k and of top-p against a sort in float64: flat rows (most of the row stays under top-p),
    peaked rows (a handful stays), ties at the k-th value, k above and below the in-kernel list."""
    g = torch.Generator().manual_seed(vocab)
    flat = torch.randn(vocab, generator=g)
    peaked = torch.randn(vocab, generator=g) * 6
    tied = flat.clone()
    tied[torch.randperm(vocab, generator=g)[:40]] = flat.max() + 1      # forty equal largest logits
    many = flat.clone()
    many[: vocab // 2] = 2.0                                            # half the row equal, near the top
    rows = torch.stack([flat, peaked, tied, many]).to(DEV).contiguous()
    for T, k, p in [(1.0, 20, 0.0), (0.7, 20, 0.95), (1.0, -1, 0.9), (0.6, -1, 0.5), (1.3, 700 if vocab <= 1000 else 5000, 0.8),
                    (1.0, 1, 0.0), (1.0, -1, 1e-6)]:
        got = _threshold_values(ops, rows, T, k, p)
        for r in range(rows.shape[0]):
            x = rows[r].cpu().double().numpy()
            order = np.sort(x)[::-1]
            kept = order
            if 0 < k < vocab:
                kept = order[order >= order[k - 1]]
            lo = hi = kept[-1]
            if 0 < p < 1:
                w = np.exp((kept - kept[0]) / T)
                c = np.cumsum(w)
                # float32 weights and a mass in fixed point move the crossing by a token or two when p falls near a step
                j_lo = int(np.searchsorted(c, (p - 2e-5) * c[-1], side="left"))
                j_hi = int(np.searchsorted(c, (p + 2e-5) * c[-1], side="left"))
                hi, lo = kept[min(j_lo, len(kept) - 1)], kept[min(j_hi, len(kept) - 1)]
            assert lo <= got[r] <= hi, (vocab, T, k, p, r, got[r], lo, hi)
            if not (0 < p < 1):
                assert got[r] == np.float32(kept[-1])


GEMM_SHAPES = [
    # M, N, K  (M <= 128: weights on the accumulator rows, K possibly cut in slices; else tokens on the rows)
    (1, 128, 64), (8, 6144, 4096), (3, 200, 72), (16, 1000, 264), (17, 333, 1024), (64, 4096, 14336),
    (100, 130, 520), (128, 256, 128), (129, 256, 128), (300, 1000, 264), (2048, 512, 1024), (513, 777, 4096),
]


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_tcgen05_gemm(ops, M, N, K, out_dtype):
    g = torch.Generator(device=DEV).manual_seed(M * 7 + N)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    got = ops.gemm_tc(x, w, out_dtype)
    torch.cuda.synchronize()
    ops.check_status()
    want = x.float() @ w.float().T
    if out_dtype == torch.float32:
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    else:
        torch.testing.assert_close(got.float(), want.bfloat16().float(), rtol=2e-2, atol=2e-2)
    # the same rows give the same bits whatever else is in the batch, as long as the tiling is the same
    again = ops.gemm_tc(x, w, out_dtype)
    assert torch.equal(got, again)


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (8, 14336, 4096), (5, 192, 72), (64, 256, 96), (128, 128, 264),
                                   (300, 320, 128), (2048, 1024, 512), (3, 176, 64), (200, 1000, 96)])
def test_gate_up_gemm_with_the_activation_in_its_epilogue(ops, M, I, K):
    g = torch.Generator(device=DEV).manual_seed(M + I)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    wg = (torch.randn(I, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    wu = (torch.randn(I, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    w13 = ops.interleave_gate_up(wg, wu)
    assert torch.equal(w13[:8], wg[:8]) and torch.equal(w13[8:16], wu[:8]) and torch.equal(w13[16:24], wg[8:16])
    got = ops.linear_glu(x, w13)
    torch.cuda.synchronize()
    ops.check_status()
    gate, up = x.float() @ wg.float().T, x.float() @ wu.float().T
    want = gate * torch.sigmoid(gate) * up
    assert got.shape == (M, I)
    torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2)
    for mode in ("all", "none"):                      # both the fused epilogue and GEMM + activation kernel
        old, ops.TC_GEMM = ops.TC_GEMM, mode
        try:
            torch.testing.assert_close(ops.linear_glu(x, w13).float(), want, rtol=3e-2, atol=3e-2)
        finally:
            ops.TC_GEMM = old
    ops.check_status()


def test_silu_mul_layouts(ops):
    g = torch.Generator(device=DEV).manual_seed(3)
    for dtype in (torch.float32, torch.bfloat16):
        gate = (torch.randn(7, 192, device=DEV, generator=g) * 3).to(dtype)
        up = torch.randn(7, 192, device=DEV, generator=g).to(dtype)
        want = (gate.float() * torch.sigmoid(gate.float()) * up.float()).to(dtype)
        halves = torch.cat([gate, up], dim=1).contiguous()
        grouped = torch.stack([gate.view(7, 3, 64), up.view(7, 3, 64)], dim=2).reshape(7, 384).contiguous()
        eights = torch.stack([gate.view(7, 24, 8), up.view(7, 24, 8)], dim=2).reshape(7, 384).contiguous()
        for u, group in ((halves, 0), (grouped, 64), (eights, 8)):
            out = torch.empty(7, 192, device=DEV, dtype=dtype)
            ops.silu_mul(u, out, group)
            torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


def test_tcgen05_gemm_rejects_what_it_cannot_do(ops):
    x = torch.zeros(4, 20, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(8, 20, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(Exception, match="multiple of 8"):
        ops.gemm_tc(x, w, torch.bfloat16)
    got = ops.linear(x, w)                      # the general entry point still serves such a width
    assert got.shape == (4, 8)
