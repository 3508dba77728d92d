"""The engine on the GPU beyond replay: each part alone, long decoding, the first
tokens of a sequence, greedy and temperature generation through the entry points,
captured decode steps against plain ones, preemption under page pressure, and a
toy mixer with state of its own that is registered from here."""
import json
import math
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = Path(__file__).resolve().parent.parent


def engine_for(folder, dtype, page, max_batch=4, max_seq=256, **kw):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_batch, max_seq_length=max_seq, page_size=page, **kw)
    return eng


# ------------------------------------------------------------------ parts alone

def _runtime(dtype):
    from batchspec_b200.parts import Runtime
    return Runtime(dtype, DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_part_rmsnorm(dtype):
    from batchspec_b200.parts import NORMS, PartSpec, build_part
    part = build_part(NORMS, PartSpec("rmsnorm", dict(dim=200, eps=3e-4)), _runtime(dtype))
    assert part.param_specs()["weight"].shape == (200,)
    g = torch.Generator(device=DEV).manual_seed(0)
    w = (1 + 0.2 * torch.randn(200, device=DEV, generator=g)).to(dtype)
    part.bind({"weight": w})
    resid = torch.randn(6, 200, device=DEV, generator=g)
    delta = torch.randn(6, 200, device=DEV, generator=g).to(dtype)
    want = P.rms_norm((resid + delta.float()).cpu(), w.float().cpu(), 3e-4)
    got = part.forward(resid, delta)
    assert got.dtype == dtype
    assert H.rel_err(got.float().cpu().numpy(), want.numpy()) <= H.TOL[str(dtype).replace("torch.", "")]


def test_part_rope_matches_the_interleaved_reference_on_permuted_rows():
    from batchspec_b200.parts import POSITION_ENCODINGS, PartSpec, build_part
    cfg = dict(H.TINY_B)
    sc = dict(cfg["rope_scaling"])
    part = build_part(POSITION_ENCODINGS, PartSpec("rope", dict(head_dim=32, theta=cfg["rope_theta"], scaling=sc)),
                      _runtime(torch.float32))
    torch.testing.assert_close(part.frequencies, P.rope_frequencies(cfg), rtol=1e-13, atol=0)
    torch.testing.assert_close(part.inv_freq.cpu().double().sum(0), P.rope_frequencies(cfg), rtol=1e-13, atol=0)
    g = torch.Generator().manual_seed(1)
    Hn, hd, T = 3, 32, 5
    w = torch.randn(Hn * hd, 24, generator=g, dtype=torch.float64)
    x = torch.randn(T, 24, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 3, 64, 65, 200])
    want = P.rope_interleaved((x @ P.permute_for_interleaved_rope(w, Hn, hd).T).reshape(T, Hn, hd), pos,
                              P.rope_frequencies(cfg))
    q = (x @ w.T).float().reshape(T, Hn, hd).to(DEV).contiguous()
    k = q[:, :1].clone()
    part.apply(q, k, SimpleNamespace(positions=pos.to(DEV, torch.int32)))
    got = q.cpu().double()
    # half-split result, re-ordered like the reference's permutation, equals the interleaved rotation
    torch.testing.assert_close(got[..., :hd // 2], want[..., 0::2], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(got[..., hd // 2:], want[..., 1::2], rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(k.cpu().double(), got[:, :1], rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_part_swiglu(dtype):
    from batchspec_b200.parts import FEED_FORWARDS, PartSpec, build_part
    part = build_part(FEED_FORWARDS, PartSpec("swiglu", dict(dim=72, intermediate=200)), _runtime(dtype))
    g = torch.Generator().manual_seed(2)
    ws = {n: (torch.randn(*s.shape, generator=g) * 0.2).to(dtype) for n, s in part.param_specs().items()}
    part.bind({n: t.to(DEV) for n, t in ws.items()})
    x = torch.randn(9, 72, generator=g).to(dtype)
    want = P.swiglu(x.double(), torch.cat([ws["gate"], ws["up"]]).double(), ws["down"].double())
    got = part.forward(x.to(DEV), None).float().cpu().double()
    assert H.rel_err(got.numpy(), want.numpy()) <= H.TOL[str(dtype).replace("torch.", "")]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 6])
def test_part_attention_and_block(dtype, window):
    """The attention part (and a whole pre-norm block around it) over a hand-made
    cache, two requests cut in two steps, against the plain functions."""
    from batchspec_b200.cache import CacheManager
    from batchspec_b200.engine.step import StepEntry, StepRunner
    from batchspec_b200.models.decoder import CacheNeed
    from batchspec_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, PartSpec, build_part
    rt = _runtime(dtype)
    d, Hq, Hkv, hd, inter = 48, 6, 2, 16, 80
    pos_spec = PartSpec("rope", dict(head_dim=hd, theta=1000.0))
    mixer = build_part(MIXERS, PartSpec("attention", dict(dim=d, n_heads=Hq, n_kv_heads=Hkv, head_dim=hd,
                                                          position=pos_spec, window=window)), rt)
    norm1 = build_part(NORMS, PartSpec("rmsnorm", dict(dim=d, eps=1e-5)), rt)
    norm2 = build_part(NORMS, PartSpec("rmsnorm", dict(dim=d, eps=1e-5)), rt)
    ffn = build_part(FEED_FORWARDS, PartSpec("swiglu", dict(dim=d, intermediate=inter)), rt)
    g = torch.Generator().manual_seed(3)
    rnd = lambda shape, s=0.3: (torch.randn(*shape, generator=g) * s).to(dtype)
    wm = {n: rnd(s.shape) for n, s in mixer.param_specs().items()}
    wf = {n: rnd(s.shape) for n, s in ffn.param_specs().items()}
    wn1, wn2 = (1 + rnd((d,), 0.1)), (1 + rnd((d,), 0.1))
    mixer.bind({n: t.to(DEV) for n, t in wm.items()})
    ffn.bind({n: t.to(DEV) for n, t in wf.items()})
    norm1.bind({"weight": wn1.to(DEV)})
    norm2.bind({"weight": wn2.to(DEV)})
    block = BLOCKS["prenorm"](norm1=norm1, mixer=mixer, norm2=norm2, ffn=ffn)
    cache = CacheManager([CacheNeed(mixer.cache_spec(), None, None)], 4, 16, 2, dtype, DEV)
    runner = StepRunner(None, cache, 10, DEV)
    xs = {"a": torch.randn(11, d, generator=g), "b": torch.randn(7, d, generator=g)}
    got = {k: [] for k in xs}
    cache.admit("a"), cache.admit("b")
    for cut in [dict(a=(0, 8), b=(0, 2)), dict(a=(8, 11), b=(2, 7))]:
        entries = [StepEntry(r, [0] * (e - b), ()) for r, (b, e) in cut.items()]
        for en in entries:
            cache.reserve(en.req_id, len(en.tokens))
        ctx = runner.build_context(entries)
        resid = torch.cat([xs[r][b:e] for r, (b, e) in cut.items()]).to(DEV).contiguous()
        resid, pending = block.forward(resid, None, ctx, cache.layer_caches[0])
        y = (resid + pending.float()).cpu()
        o = 0
        for r, (b, e) in cut.items():
            got[r].append(y[o:o + e - b])
            o += e - b
            cache.commit(r, e - b)
    for r, x in xs.items():
        x = x.double()
        T = x.shape[0]
        a = P.rms_norm(x, wn1.double(), 1e-5)
        q = (a @ wm["q"].double().T).reshape(T, Hq, hd)
        k = (a @ wm["k"].double().T).reshape(T, Hkv, hd)
        v = (a @ wm["v"].double().T).reshape(T, Hkv, hd)
        f = 1000.0 ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)
        def rot(t):        # half-split pairing, as the part does on un-permuted rows
            ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None]
            c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
            lo, hi = t[..., :hd // 2], t[..., hd // 2:]
            return torch.cat([lo * c - hi * s, lo * s + hi * c], -1)
        att = P.causal_attention(rot(q), rot(k), v, window=window).reshape(T, Hq * hd) @ wm["o"].double().T
        h = x + att
        want = h + P.swiglu(P.rms_norm(h, wn2.double(), 1e-5), torch.cat([wf["gate"], wf["up"]]).double(),
                            wf["down"].double())
        assert H.rel_err(torch.cat(got[r]).numpy(), want.numpy()) <= H.TOL[str(dtype).replace("torch.", "")]
    if window:
        assert cache.requests["a"].tables[0][0] == -1, "pages behind the window were given back"


# ------------------------------------------------------------------ whole engine

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    """Positions 0, 1, 2: one key, no history, a page's first rows."""
    cfg, seed, page = H.TINY["A"]
    folder = H.make_folder(tmp_path, cfg, seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    eng = engine_for(folder, dtype, page)
    for n in (1, 2, 3):
        toks = H.random_tokens(n, cfg["vocab_size"], 40 + n)
        for sched in (H.whole("x", toks), H.portions("x", toks, [1])):
            H.compare_with_oracle(H.run_steps_in_process(eng, sched), folder, {"x": toks}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_token_by_token(tmp_path, dtype):
    """A short prompt and 200 single-token steps: every page edge is crossed by a
    decode step, the split-key kernel sees every length."""
    cfg, seed, _ = H.TINY["C"]
    folder = H.make_folder(tmp_path, cfg, seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    eng = engine_for(folder, dtype, 16, max_seq=256)
    toks = H.random_tokens(210, cfg["vocab_size"], 77)
    got = H.run_steps_in_process(eng, H.tail_decoded("x", toks, tail=200))
    H.compare_with_oracle(got, folder, {"x": toks}, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY[name]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    cfg, w = P.read_model_folder(folder)
    lens = [5, 17, 33] if name == "A" else [1, 9, 40, 64, 130]
    prompts = [H.random_tokens(n, cfgj["vocab_size"], 7 * n) for n in lens]
    eng = engine_for(folder, dtype, page, max_batch=3, max_seq=cfgj["max_position_embeddings"], prefill_chunk_size=16,
                     max_tokens_per_step=24)
    eng.setup_sampling_params(temperature=0.0)
    done = {s.seq_id: s for s in eng.generate([Sequence(i, p, max_new_tokens=8) for i, p in enumerate(prompts)])}
    assert len(done) == len(prompts)
    for i, p in enumerate(prompts):
        out = done[i].output_ids
        assert len(out) == 8 and done[i].finish_reason == "length"
        ref = P.forward(cfg, w, p + out[:-1])
        scale = float(ref.abs().max())
        for k, tok in enumerate(out):                       # the oracle's argmax, or a tie within the tolerance
            row = ref[len(p) - 1 + k]
            assert float(row.max() - row[tok]) <= H.TOL[dtype] * scale, (i, k, tok, int(row.argmax()))
        if dtype == "float32":
            assert out == P.greedy_generate(cfg, w, p, 8)
    assert eng.cache.groups[0].pool.num_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps_equal_plain_ones(tmp_path, dtype):
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY["C"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    prompts = [H.random_tokens(n, cfgj["vocab_size"], n) for n in (30, 4, 61)]
    outs = {}
    for graphs in (False, True):
        eng = engine_for(folder, dtype, page, max_batch=3, max_seq=128, prefill_chunk_size=64, max_tokens_per_step=128)
        eng.use_cuda_graphs = graphs
        eng.setup_sampling_params(temperature=0.7, top_k=40, top_p=0.9, seed=5)
        done = eng.generate([Sequence(i, p, max_new_tokens=40) for i, p in enumerate(prompts)])
        outs[graphs] = {s.seq_id: s.output_ids for s in done}
        if graphs:
            assert any(g.graph is not None for g in eng._graphs.values()), "no decode step was captured"
            # the same generation with every captured step timed on the device: same tokens, one time per decode
            # step; in sum no longer than the steps' wall time (a step launched ahead starts inside the wall time
            # of the step before it, so the two are not comparable step by step)
            eng.time_decode_on_device = True
            again = eng.generate([Sequence(i, p, max_new_tokens=40) for i, p in enumerate(prompts)])
            assert {s.seq_id: s.output_ids for s in again} == outs[True]
            st = eng.last_stats
            assert len(st["decode_step_device_ms"]) == len(st["decode_step_ms"]) > 0
            assert all(d > 0.0 for d in st["decode_step_device_ms"])
            assert sum(st["decode_step_device_ms"]) <= sum(st["decode_step_ms"]) + 0.1
    assert outs[True] == outs[False]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_launched_ahead_change_nothing(tmp_path, dtype):
    """The engine launches the next captured decode step before it has read the current one's tokens.  Requests
    that end on an end-of-sequence token (which only the GPU knows when the step ahead is launched), on their token
    limit or on the context limit, more requests than fit at once (so that others are admitted when one ends) and
    different lengths must give exactly the tokens of an engine that does not look ahead."""
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY["C"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32 if dtype == "float32" else torch.bfloat16)
    prompts = [H.random_tokens(n, cfgj["vocab_size"], 7 * n + 1) for n in (30, 4, 61, 12, 33, 5, 90)]
    limits = [40, 3, 25, 60, 1, 17, 50]
    def run(ahead, eos, count=None):
        eng = engine_for(folder, dtype, page, max_batch=4, max_seq=120, prefill_chunk_size=64, max_tokens_per_step=128)
        eng.decode_lookahead = ahead
        eng.setup_sampling_params(temperature=0.9, top_k=50, seed=3)
        eng.setup_special_tokens(eos_token_ids=eos)
        if count is not None:
            real = eng._launch_decode
            def counting(graph, seqs, tokens, is_ahead):
                count[0] += int(is_ahead)
                return real(graph, seqs, tokens, is_ahead)
            eng._launch_decode = counting
        done = eng.generate([Sequence(i, p, max_new_tokens=m) for i, (p, m) in enumerate(zip(prompts, limits))])
        eng.cache.check_invariants()
        return {s.seq_id: s.output_ids for s in done}, {s.seq_id: s.finish_reason for s in done}

    # end-of-sequence tokens that do turn up: what requests 0, 2 and 3 draw a third of the way in
    free, _ = run(False, [])
    eos = sorted({free[i][len(free[i]) // 3] for i in (0, 2, 3)})
    outs, reasons, count = {}, {}, [0]
    for ahead in (False, True):
        outs[ahead], reasons[ahead] = run(ahead, eos, count if ahead else None)
    launched_ahead = count[0]
    assert outs[True] == outs[False] and reasons[True] == reasons[False]
    assert launched_ahead > 10, "no step was launched ahead"
    assert "eos" in reasons[True].values() and "length" in reasons[True].values()


def test_temperature_sampling_does_not_depend_on_the_schedule(tmp_path):
    """Config B's workload: five prompts, chunks of 16 mixed with decode steps,
    temperature 0.8 under a fixed seed: the same tokens whatever the batching."""
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY["B"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32)
    prompts = [H.random_tokens(n, cfgj["vocab_size"], 3 * n) for n in (1, 9, 40, 64, 130)]
    results = []
    for max_batch, chunk, budget in [(5, 16, 40), (2, 16, 16), (1, 256, 256), (5, 7, 9)]:
        eng = engine_for(folder, "float32", page, max_batch=max_batch, max_seq=256, prefill_chunk_size=chunk,
                         max_tokens_per_step=budget)
        eng.setup_sampling_params(temperature=0.8, seed=11)
        done = eng.generate([Sequence(i, p, max_new_tokens=12) for i, p in enumerate(prompts)])
        results.append({s.seq_id: s.output_ids for s in done})
    assert all(r == results[0] for r in results[1:])
    assert len({tuple(v) for v in results[0].values()}) == 5


def test_preemption_under_page_pressure_changes_nothing(tmp_path):
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY["A"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32)
    prompts = [H.random_tokens(n, cfgj["vocab_size"], 11 * n) for n in (20, 25, 30, 18)]
    outs = []
    for num_pages in (64, 22):                       # roomy, then too small for all four at their full length
        eng = engine_for(folder, "float32", page, max_batch=4, max_seq=128, prefill_chunk_size=32,
                         max_tokens_per_step=64, num_pages=num_pages)
        eng.setup_sampling_params(temperature=0.0)
        done = eng.generate([Sequence(i, p, max_new_tokens=30) for i, p in enumerate(prompts)])
        outs.append({s.seq_id: s.output_ids for s in done})
        if num_pages == 22:
            assert eng.last_stats["preemptions"] >= 1
        assert eng.cache.groups[0].pool.num_held == 0
    assert outs[0] == outs[1]


def test_everything_at_once_gives_the_same_tokens(tmp_path):
    """Many requests of random lengths and limits, sampled, some ending on end-of-sequence tokens, more than fit at
    once, through a pool so small that requests are preempted: the tokens are those of a roomy engine without
    captured graphs, whether decode steps are captured or not and launched ahead or not (float32: every kernel
    then gives a row the same bits whatever else is in the step)."""
    import random
    from batchspec_b200.engine import Sequence
    cfgj, seed, page = H.TINY["A"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32)
    rng = random.Random(4)
    prompts = [H.random_tokens(rng.randint(1, 70), cfgj["vocab_size"], 100 + i) for i in range(14)]
    limits = [rng.randint(1, 45) for _ in prompts]

    def run(num_pages, graphs, ahead, eos):
        eng = engine_for(folder, "float32", page, max_batch=5, max_seq=128, prefill_chunk_size=24,
                         max_tokens_per_step=48, num_pages=num_pages)
        eng.use_cuda_graphs, eng.decode_lookahead = graphs, ahead
        eng.setup_sampling_params(temperature=0.8, top_k=30, top_p=0.9, seed=21)
        eng.setup_special_tokens(eos_token_ids=eos)
        done = eng.generate([Sequence(i, p, max_new_tokens=m) for i, (p, m) in enumerate(zip(prompts, limits))])
        eng.cache.check_invariants()
        assert all(g.pool.num_held == 0 for g in eng.cache.groups)
        H.assert_unused_pages_untouched(eng)        # (the roomy runs leave most of their 400 pages unused)
        return ({s.seq_id: s.output_ids for s in done}, {s.seq_id: s.finish_reason for s in done},
                eng.last_stats["preemptions"])

    free, _, _ = run(400, False, False, [])
    eos = sorted({free[i][len(free[i]) // 2] for i in (1, 4, 7, 10) if len(free[i]) > 3})
    want = run(400, False, False, eos)
    assert "eos" in want[1].values() and "length" in want[1].values()
    tight = -(-max(len(p) + m for p, m in zip(prompts, limits)) // page) + 8       # the longest request and little more
    preempted = 0
    for graphs, ahead in [(False, False), (True, False), (True, True)]:
        got = run(tight, graphs, ahead, eos)
        for i in want[0]:
            assert got[0][i] == want[0][i], (graphs, ahead, i, len(prompts[i]), limits[i], got[2],
                                             [k for k, (a, b) in enumerate(zip(got[0][i], want[0][i])) if a != b][:3],
                                             len(got[0][i]), len(want[0][i]))
        assert got[1] == want[1], (graphs, ahead)
        preempted += got[2]
    assert preempted >= 3, "the small pool never forced a preemption"


def test_prompts_held_up_for_pages_beside_a_step_launched_ahead(tmp_path):
    """Two requests decode while two more, admitted but in the middle of their prompts, get no pages; one of the
    decoding ones ends on an end-of-sequence token that only the GPU knows when the next step has already been
    launched ahead.  The step after that feeds prompt portions again, so the step launched ahead stands for nothing:
    it must neither be launched in that situation nor be taken for a later step."""
    from batchspec_b200.engine import Sequence
    cfgj, seed, _ = H.TINY["B"]
    page = 16
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.float32)
    lens, limits = [6, 96, 43, 15, 1, 104, 38, 83], [9, 25, 6, 3, 37, 4, 4, 10]
    prompts = [H.random_tokens(n, cfgj["vocab_size"], 15600 + i) for i, n in enumerate(lens)]

    def run(num_pages, graphs, ahead, eos):
        eng = engine_for(folder, "float32", page, max_batch=5, max_seq=128, prefill_chunk_size=16,
                         max_tokens_per_step=32, num_pages=num_pages)
        eng.use_cuda_graphs, eng.decode_lookahead = graphs, ahead
        eng.setup_sampling_params(temperature=0.9, top_k=5, top_p=0.9, seed=156)
        eng.setup_special_tokens(eos_token_ids=eos)
        done = eng.generate([Sequence(i, p, max_new_tokens=m) for i, (p, m) in enumerate(zip(prompts, limits))])
        eng.cache.check_invariants()
        return {s.seq_id: s.output_ids for s in done}, eng.last_stats["preemptions"]

    free, _ = run(400, False, False, [])
    eos = sorted({free[i][len(free[i]) // 2] for i in (0, 3, 6) if len(free[i]) > 3})
    want, _ = run(400, False, False, eos)
    got, preempted = run(9, True, True, eos)
    assert preempted >= 1
    assert got == want


@pytest.mark.parametrize("graphs", [False, True])
def test_a_wait_given_up_is_reported_not_taken_for_a_result(tmp_path, graphs):
    """Kernels bound their waits and record a code in a status word when they give one up.  The engine looks at that
    word whenever it reads a step's tokens.  The word is set by hand here (no kernel is made to wait in vain): the
    next read raises instead of returning tokens, and afterwards the engine works as before."""
    from batchspec_b200.engine import Sequence
    from batchspec_b200.kernels import ops
    cfgj, seed, page = H.TINY["C"]
    folder = H.make_folder(tmp_path, cfgj, seed, dtype=torch.bfloat16)
    eng = engine_for(folder, "bfloat16", page, max_batch=2, max_seq=64)
    eng.use_cuda_graphs = graphs
    eng.setup_sampling_params(temperature=0.0)
    prompts = [H.random_tokens(9, cfgj["vocab_size"], 3), H.random_tokens(14, cfgj["vocab_size"], 4)]

    def run():
        return [s.output_ids for s in sorted(eng.generate([Sequence(i, p, max_new_tokens=6)
                                                            for i, p in enumerate(prompts)]), key=lambda s: s.seq_id)]
    want = run()
    with torch.inference_mode():          # the word was made inside a step, which runs in inference mode
        ops._status_word(torch.device(DEV)).fill_(12)
    with pytest.raises(ops.KernelError, match="code 12"):
        run()
    assert run() == want


def test_command_line_entry_point(tmp_path):
    cfgj, seed, page = H.TINY["A"]
    folder = H.make_folder(tmp_path / "m", cfgj, seed, dtype=torch.bfloat16)
    cmd = [sys.executable, "-m", "batchspec_b200.run_e2e", "--checkpoint_path", str(folder), "--batch_size", "3",
           "--prefix_len", "20", "--max_gen_len", "6", "--temperature", "0.0", "--page_size", str(page),
           "--printoutput", "--force_budget", "--profiling", "--prof_output_dir", str(tmp_path / "prof")]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Total generated tokens: 18" in r.stdout and "--- sequence 2" in r.stdout
    summary = json.loads((tmp_path / "prof" / "run" / "summary.json").read_text())
    assert summary["step_ms"]["count"] >= 6 and "attn.compute" in summary["buckets_ms"]


def test_benchmark_entry_point(tmp_path):
    cfgj, seed, page = H.TINY["C"]
    folder = H.make_folder(tmp_path / "m", cfgj, seed, dtype=torch.bfloat16)
    cmd = [sys.executable, "-m", "batchspec_b200.run_benchmark", "--checkpoint_path", str(folder), "--batch_size", "4",
           "--prefix_len_list", "24", "70", "--max_gen_len", "10", "--num_total_runs", "3", "--temperature", "0.6",
           "--top_k", "20", "--top_p", "0.95", "--force_budget", "--profiling", "--model_profiling", "false",
           "--prof_output_dir", str(tmp_path / "prof")]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "prefix 24:" in r.stdout and "prefix 70:" in r.stdout
    for prefix in (24, 70):
        summary = json.loads((tmp_path / "prof" / f"bench-bsz4-prefix{prefix}-gen10" / "summary.json").read_text())
        assert summary["throughput_tok_s"] > 0 and summary["runs"] == 3 and summary["warmup_runs"] == 1


# ------------------------------------------------------------------ a toy mixer with state, registered from the test

def test_a_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """An architecture defined here: layers alternate a recurrent toy mixer (state
    s_t = decay * s_{t-1} + x_t per request, output s_t W^T) with the framework's
    attention.  It is registered, built from a config.json, given random weights
    and stepped whole, in portions and mixed, with no change to the framework."""
    from dataclasses import dataclass
    from batchspec_b200.config import config_from_json_dict, register_config_class
    from batchspec_b200.engine import Engine
    from batchspec_b200.models import ModelSpec, prenorm_layer, RunEntry, register_model
    from batchspec_b200.parts import MIXERS, Mixer, ParamSpec, PartSpec, StateSpec, register_part

    @register_part(MIXERS, "toy_decay")
    class ToyDecay(Mixer):
        def __init__(self, runtime, dim, decay):
            self.runtime, self.dim, self.decay = runtime, dim, decay

        def param_specs(self):
            return {"w": ParamSpec((self.dim, self.dim))}

        def bind(self, params):
            self.w = params["w"].float()

        def state_spec(self):
            return StateSpec((self.dim,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            for e in range(ctx.n_entries):
                b, en, slot = int(ctx.h_qo_indptr[e]), int(ctx.h_qo_indptr[e + 1]), int(ctx.h_state_slots[e])
                s = cache.state[slot].clone()
                for t in range(b, en):
                    s = self.decay * s + x[t].float()
                    out[t] = (self.w @ s).to(x.dtype)
                cache.state[slot] = s
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        architecture: str
        vocab_size: int
        width: int
        depth: int
        decay: float
        eps: float

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["width"], d["depth"], d["decay"], d["eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, width=self.width,
                        depth=self.depth, decay=self.decay, eps=self.eps)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.eps))
        toy = PartSpec("toy_decay", dict(dim=cfg.width, decay=cfg.decay))
        att = PartSpec("attention", dict(dim=cfg.width, n_heads=2, n_kv_heads=1, head_dim=16,
                                         position=PartSpec("rope", dict(head_dim=16, theta=100.0))))
        ffn = PartSpec("swiglu", dict(dim=cfg.width, intermediate=2 * cfg.width))
        layers = []
        for i in range(cfg.depth):
            names = {"norm1.weight": f"l{i}.n1", "norm2.weight": f"l{i}.n2", "ffn.gate": f"l{i}.gate",
                     "ffn.up": f"l{i}.up", "ffn.down": f"l{i}.down"}
            if i % 2 == 0:
                names["mixer.w"] = f"l{i}.toy"
                layers.append(prenorm_layer(norm, toy, norm, ffn, names))
            else:
                names.update({"mixer." + k: f"l{i}.{k}" for k in "qkvo"})
                layers.append(prenorm_layer(norm, att, norm, ffn, names))
        return ModelSpec(cfg.vocab_size, cfg.width, layers, [RunEntry(i) for i in range(cfg.depth)], norm,
                         "emb", {"weight": "final"}, None)

    register_config_class("ToyStateLM", ToyConfig)
    register_model("ToyStateLM", build)
    cfg = config_from_json_dict(dict(architectures=["ToyStateLM"], vocab_size=61, width=24, depth=3, decay=0.5, eps=1e-5))
    from batchspec_b200.weights import write_random_model
    folder = write_random_model(cfg, tmp_path, seed=4, dtype=torch.float32, std=0.2, norm_std=0.1)
    _, w = P.read_model_folder(folder)

    def oracle(tokens):
        x = w["emb"][torch.tensor(tokens)]
        T = len(tokens)
        for i in range(cfg.depth):
            a = P.rms_norm(x, w[f"l{i}.n1"], cfg.eps)
            if i % 2 == 0:
                s, ys = torch.zeros(cfg.width, dtype=torch.float64), []
                for t in range(T):
                    s = cfg.decay * s + a[t]
                    ys.append(w[f"l{i}.toy"] @ s)
                y = torch.stack(ys)
            else:
                f = 100.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
                ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None]
                c, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
                rot = lambda t: torch.cat([t[..., :8] * c - t[..., 8:] * sn, t[..., :8] * sn + t[..., 8:] * c], -1)
                q = rot((a @ w[f"l{i}.q"].T).reshape(T, 2, 16))
                k = rot((a @ w[f"l{i}.k"].T).reshape(T, 1, 16))
                v = (a @ w[f"l{i}.v"].T).reshape(T, 1, 16)
                y = P.causal_attention(q, k, v).reshape(T, 32) @ w[f"l{i}.o"].T
            h = x + y
            x = h + P.swiglu(P.rms_norm(h, w[f"l{i}.n2"], cfg.eps), torch.cat([w[f"l{i}.gate"], w[f"l{i}.up"]]),
                             w[f"l{i}.down"])
        return (P.rms_norm(x, w["final"], cfg.eps) @ w["emb"].T).numpy()

    eng = Engine(dtype="float32", device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=2, max_seq_length=64, page_size=4, num_pages=24)
    assert eng.decode_graph(2) is None, "a host-driven mixer must keep decode steps out of CUDA graphs"
    needs = eng.model.cache_needs()
    assert needs[0].state is not None and needs[0].cache is None and needs[1].cache is not None
    reqs = {f"t{i}": H.random_tokens(n, 61, 50 + i) for i, n in enumerate((9, 14, 5, 11))}
    for rid, toks in reqs.items():
        for sched in (H.whole(rid, toks), H.portions(rid, toks, [3, 2, 5])):
            got = H.run_steps_in_process(eng, sched)
            for p_ in range(len(toks)):
                assert H.rel_err(got[(rid, p_)], oracle(toks)[p_]) <= H.TOL["float32"]
    got = H.run_steps_in_process(eng, H.mixed(reqs, seed=1, max_live=2))       # state slots are reused
    for rid, toks in reqs.items():
        ref = oracle(toks)
        for p_ in range(len(toks)):
            assert H.rel_err(got[(rid, p_)], ref[p_]) <= H.TOL["float32"], (rid, p_)


# ------------------------------------- run order as data; a routed feed-forward and another position encoding as toys

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_shared_cache_window_and_toy_parts(tmp_path, dtype):
    """An architecture defined here, with everything the model description allows at once: two layers run four
    times (layer 0, layer 1, layer 0 again with a cache of its own, layer 1 again reading the cache its first run
    wrote); layer 1's attention sees a window of 5 keys (so its pages are a pool of their own and are given back
    as the window passes) and uses a position encoding registered here (no rotation: q and k are scaled by
    exp(+-rate * dim * position), which makes scores depend on distance); layer 1's feed-forward is a routed toy
    registered here (router logits in 32-bit, the best 2 of 3 experts, weights renormalised; see TOPK).  Stepped whole, in
    portions and mixed with reused pages and compared with an oracle written out below."""
    from dataclasses import dataclass
    from batchspec_b200.config import config_from_json_dict, register_config_class
    from batchspec_b200.engine import Engine
    from batchspec_b200.models import ModelSpec, prenorm_layer, RunEntry, register_model
    from batchspec_b200.parts import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, ParamSpec, PartSpec,
                                      PositionEncoding, register_part)
    from batchspec_b200.weights import write_random_model

    W, HD, HQ, HKV, WINDOW, RATE, E, INNER = 32, 16, 2, 1, 5, 0.004, 3, 24
    # the best 2 of 3 experts in 32-bit; in bfloat16 all 3 are weighed, because a near tie between the second and
    # the third would flip the choice on rounding alone and the comparison with the oracle would test luck
    TOPK = 2 if dtype == "float32" else 3
    OUT_SCALE = 1.0

    @register_part(POSITION_ENCODINGS, "toy_distance_scale")
    class ToyDistanceScale(PositionEncoding):
        def __init__(self, runtime, head_dim, rate):
            self.runtime, self.rate = runtime, rate
            self.dims = torch.arange(head_dim, dtype=torch.float32, device=runtime.device)

        def param_specs(self):
            return {}

        def bind(self, params):
            pass

        def apply(self, q, k, ctx):
            f = torch.exp(self.rate * ctx.positions.float()[:, None, None] * self.dims)      # [n, 1, hd], 32-bit
            q.copy_((q.float() * f).to(q.dtype))
            k.copy_((k.float() / f).to(k.dtype))

    @register_part(FEED_FORWARDS, "toy_routed")
    class ToyRouted(FeedForward):
        def __init__(self, runtime, dim, inner, experts, top_k, out_scale):
            self.runtime, self.dim, self.inner, self.experts, self.top_k = runtime, dim, inner, experts, top_k
            self.out_scale = out_scale

        def param_specs(self):
            return {"router": ParamSpec((self.experts, self.dim)), "w1": ParamSpec((self.experts * self.inner, self.dim)),
                    "w2": ParamSpec((self.experts * self.dim, self.inner))}

        def bind(self, params):
            self.router = params["router"].float()
            self.w1 = params["w1"].view(self.experts, self.inner, self.dim)
            self.w2 = params["w2"].view(self.experts, self.dim, self.inner)

        def forward(self, x, ctx):
            logits = x.float() @ self.router.T                                   # 32-bit router
            top, idx = torch.topk(logits, self.top_k, dim=-1)
            gate = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.experts):
                h = torch.relu(x @ self.w1[e].T)
                y = (h @ self.w2[e].T).float()
                out += y * (gate * (idx == e)).sum(-1, keepdim=True)
            return (out * self.out_scale).to(x.dtype)

    @dataclass(frozen=True)
    class MixConfig:
        architecture: str
        vocab_size: int
        eps: float

        @classmethod
        def from_json_dict(cls, d):
            return cls(d["architectures"][0], d["vocab_size"], d["eps"])

        def to_json_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, eps=self.eps)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(dim=W, eps=cfg.eps))
        att0 = PartSpec("attention", dict(dim=W, n_heads=HQ, n_kv_heads=HKV, head_dim=HD,
                                          position=PartSpec("rope", dict(head_dim=HD, theta=100.0))))
        att1 = PartSpec("attention", dict(dim=W, n_heads=HQ, n_kv_heads=HKV, head_dim=HD, window=WINDOW,
                                          position=PartSpec("toy_distance_scale", dict(head_dim=HD, rate=RATE))))
        ffn0 = PartSpec("swiglu", dict(dim=W, intermediate=40))
        ffn1 = PartSpec("toy_routed", dict(dim=W, inner=INNER, experts=E, top_k=TOPK, out_scale=OUT_SCALE))
        names0 = {"norm1.weight": "a.n1", "norm2.weight": "a.n2", "ffn.gate": "a.gate", "ffn.up": "a.up", "ffn.down": "a.down"}
        names0.update({"mixer." + k: "a." + k for k in "qkvo"})
        names1 = {"norm1.weight": "b.n1", "norm2.weight": "b.n2", "ffn.router": "b.router", "ffn.w1": "b.w1", "ffn.w2": "b.w2"}
        names1.update({"mixer." + k: "b." + k for k in "qkvo"})
        layers = [prenorm_layer(norm, att0, norm, ffn0, names0), prenorm_layer(norm, att1, norm, ffn1, names1)]
        order = [RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(1, cache_from=1)]
        return ModelSpec(cfg.vocab_size, W, layers, order, norm, "emb", {"weight": "final"}, None)

    register_config_class("ToyMixLM", MixConfig)
    register_model("ToyMixLM", build)
    cfg = config_from_json_dict(dict(architectures=["ToyMixLM"], vocab_size=53, eps=1e-5))
    folder = write_random_model(cfg, tmp_path, seed=9, dtype=torch.float32 if dtype == "float32" else torch.bfloat16,
                                std=0.08, norm_std=0.1)
    _, w = P.read_model_folder(folder)

    def rope(t, T):
        f = 100.0 ** (-2.0 * torch.arange(HD // 2, dtype=torch.float64) / HD)
        ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None]
        c, sn = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        h = HD // 2
        return torch.cat([t[..., :h] * c - t[..., h:] * sn, t[..., :h] * sn + t[..., h:] * c], -1)

    def oracle(tokens):
        T = len(tokens)
        x = w["emb"][torch.tensor(tokens)]
        dist = torch.exp(RATE * torch.arange(T, dtype=torch.float64)[:, None, None] * torch.arange(HD, dtype=torch.float64))
        kept = {}
        for run, (layer, reads) in enumerate([("a", None), ("b", None), ("a", None), ("b", 1)]):
            a = P.rms_norm(x, w[f"{layer}.n1"], cfg.eps)
            q = (a @ w[f"{layer}.q"].T).reshape(T, HQ, HD)
            k = (a @ w[f"{layer}.k"].T).reshape(T, HKV, HD)
            v = (a @ w[f"{layer}.v"].T).reshape(T, HKV, HD)
            if layer == "a":
                q, k = rope(q, T), rope(k, T)
                window = None
            else:
                q, k = q * dist, k / dist
                window = WINDOW
            if reads is None:
                kept[run] = (k, v)
            else:
                k, v = kept[reads]                           # the keys and values its first run cached
            y = P.causal_attention(q, k, v, window=window).reshape(T, HQ * HD) @ w[f"{layer}.o"].T
            h = x + y
            n2 = P.rms_norm(h, w[f"{layer}.n2"], cfg.eps)
            if layer == "a":
                f = P.swiglu(n2, torch.cat([w["a.gate"], w["a.up"]]), w["a.down"])
            else:
                logits = n2 @ w["b.router"].T
                top, idx = torch.topk(logits, TOPK, dim=-1)
                gate = torch.softmax(top, dim=-1)
                f = torch.zeros_like(n2)
                for e in range(E):
                    w1, w2 = w["b.w1"][e * INNER:(e + 1) * INNER], w["b.w2"][e * W:(e + 1) * W]
                    f += (torch.relu(n2 @ w1.T) @ w2.T) * (gate * (idx == e)).sum(-1, keepdim=True)
                f = f * OUT_SCALE
            x = h + f
        return (P.rms_norm(x, w["final"], cfg.eps) @ w["emb"].T).numpy()

    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=3, max_seq_length=48, page_size=4, num_pages=[40, 24])
    needs = eng.model.cache_needs()
    assert [n.cache_from for n in needs] == [None, None, None, 1]
    assert len(eng.cache.groups) == 2 and [g.spec.policy for g in eng.cache.groups] == ["full", "window"]
    assert [len(g.runs) for g in eng.cache.groups] == [2, 1], "layer 0 twice owns two caches, the reader none"
    reqs = {f"m{i}": H.random_tokens(n, 53, 70 + i) for i, n in enumerate((19, 30, 7, 26))}
    tol = H.TOL[dtype]
    for rid, toks in reqs.items():
        ref = oracle(toks)
        for sched in (H.whole(rid, toks), H.portions(rid, toks, [4, 2, 7, 3])):
            got = H.run_steps_in_process(eng, sched)
            for p_ in range(len(toks)):
                assert H.rel_err(got[(rid, p_)], ref[p_]) <= tol, (rid, p_, dtype)
    got = H.run_steps_in_process(eng, H.mixed(reqs, seed=2, max_live=3))
    for rid, toks in reqs.items():
        ref = oracle(toks)
        for p_ in range(len(toks)):
            assert H.rel_err(got[(rid, p_)], ref[p_]) <= tol, (rid, p_, dtype)
    eng.cache.check_invariants()


def test_kernel_microbenchmarks_run():
    """The microbenchmarks of kernels/microbench.py on a small configuration: they use the kernels' current
    interfaces (a changed signature shows here, not on the day a profile is wanted)."""
    import subprocess
    import sys
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    out = subprocess.run([sys.executable, "-m", "batchspec_b200.kernels.microbench", "--config", "llama-3.2-1b", "--what",
                          "gemm", "attention", "small", "--m", "8", "64"], cwd=root, capture_output=True, text=True,
                         timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "add_rmsnorm" in out.stdout and "rope_kv_append" in out.stdout
