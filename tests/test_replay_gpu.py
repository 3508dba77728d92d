"""Replay on the GPU against the plain implementation: whole, tail decoded one by
one, portions of changing size, and mixed requests on a pool so small that pages
are used again; in float32 and bfloat16, on the tiny configurations."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 40, 64, 130], "C": [3, 50, 131, 200]}


def _folder(tmp_path, name, dtype):
    cfg, seed, _ = H.TINY[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    return H.make_folder(tmp_path / f"{name}_{dtype}", cfg, seed, dtype=stored)


def _engine(folder, dtype, page_size, num_pages, max_requests=8):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_requests, page_size=page_size, num_pages=num_pages)
    return eng


def _requests(name):
    cfg, seed, _ = H.TINY[name]
    return {f"r{i}": H.random_tokens(n, cfg["vocab_size"], 100 * seed + i) for i, n in enumerate(LENGTHS[name])}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_tail_portions(tmp_path, name, dtype):
    cfg, seed, page = H.TINY[name]
    folder = _folder(tmp_path, name, dtype)
    reqs = _requests(name)
    longest = max(len(t) for t in reqs.values())
    eng = _engine(folder, dtype, page, -(-longest // page) + 1)
    for rid, toks in reqs.items():
        one = {rid: toks}
        got = H.run_steps_in_process(eng, H.whole(rid, toks))
        H.compare_with_oracle(got, folder, one, dtype)
        got_tail = H.run_steps_in_process(eng, H.tail_decoded(rid, toks, tail=32))
        H.compare_with_oracle(got_tail, folder, one, dtype)
        got_port = H.run_steps_in_process(eng, H.portions(rid, toks, [7, 2, 16, 3, 2, 5, 2, 31]))
        H.compare_with_oracle(got_port, folder, one, dtype)
        assert set(got) == set(got_tail) == set(got_port)
        # the ways of cutting agree with each other more closely than with the oracle
        for key in got:
            scale = np.abs(got[key]).max()
            lim = H.TOL[dtype] * scale
            assert np.abs(got[key] - got_tail[key]).max() <= lim
            assert np.abs(got[key] - got_port[key]).max() <= lim
    assert eng.cache.groups[0].pool.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_requests_reuse_pages(tmp_path, name, dtype):
    cfg, seed, page = H.TINY[name]
    folder = _folder(tmp_path, name, dtype)
    base = _requests(name)
    reqs = dict(base)
    for i, (rid, toks) in enumerate(base.items()):          # twice as many requests as fit at once
        reqs[f"s{i}"] = H.random_tokens(max(2, len(toks) // 2 + 3), cfg["vocab_size"], 999 + i)
    steps = H.mixed(reqs, seed=seed + 7, max_live=4)
    max_tokens = H.max_live_tokens(steps, round_to=page)
    eng = _engine(folder, dtype, page, max_tokens // page, max_requests=4)
    got = H.run_steps_in_process(eng, steps)
    assert eng.cache.groups[0].pool.high_water <= max_tokens // page
    total_pages = sum(-(-len(t) // page) for t in reqs.values())
    assert total_pages > eng.cache.groups[0].pool.num_pages, "the schedule must force pages to be used again"
    H.compare_with_oracle(got, folder, reqs, dtype)
    assert len(got) == sum(len(t) for t in reqs.values())


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tmp_path, dtype):
    """The program itself, as a child process, on the mixed schedule of config B."""
    cfg, seed, page = H.TINY["B"]
    folder = _folder(tmp_path, "B", dtype)
    reqs = _requests("B")
    steps = H.mixed(reqs, seed=3, max_live=4)
    max_tokens = H.max_live_tokens(steps, round_to=64)
    got = H.run_trace_subprocess(folder, dtype, steps, tmp_path / "out", max_tokens)
    H.compare_with_oracle(got, folder, reqs, dtype)
    assert len(got) == sum(len(t) for t in reqs.values())


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_sizes_of_the_8b_model(tmp_path, dtype):
    """One layer at Llama-3-8B's sizes (hidden 4096, 32/8 heads of 128, intermediate 14336), page 16: whole, tail
    decoded, portions and a mixed schedule.  In bfloat16 this is where the tcgen05 GEMM (with the activation in
    its epilogue), the tcgen05 attention for long portions and the TMA split-key decode attention run inside the
    engine."""
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = H.make_folder(tmp_path / "wide", H.WIDE, 5, dtype=stored, std=0.02, norm_std=0.1)
    reqs = {"w0": H.random_tokens(300, 2048, 1), "w1": H.random_tokens(70, 2048, 2), "w2": H.random_tokens(150, 2048, 3)}
    eng = _engine(folder, dtype, 16, 40, max_requests=3)
    got = H.run_steps_in_process(eng, H.whole("w0", reqs["w0"]))
    H.compare_with_oracle(got, folder, {"w0": reqs["w0"]}, dtype)
    got = H.run_steps_in_process(eng, H.tail_decoded("w1", reqs["w1"], tail=32))
    H.compare_with_oracle(got, folder, {"w1": reqs["w1"]}, dtype)
    got = H.run_steps_in_process(eng, H.portions("w2", reqs["w2"], [40, 2, 70, 3, 20, 15]))
    H.compare_with_oracle(got, folder, {"w2": reqs["w2"]}, dtype)
    steps = H.mixed(reqs, seed=9, max_live=3, sizes=(64, 1, 2, 100, 1, 33, 1, 1))
    eng2 = _engine(folder, dtype, 16, H.max_live_tokens(steps, 16) // 16, max_requests=3)
    got = H.run_steps_in_process(eng2, steps)
    H.compare_with_oracle(got, folder, reqs, dtype)
