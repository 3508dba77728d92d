"""The model at its real width, vocabulary and depth.

* Four layers at Llama-3-8B's layer sizes with the full vocabulary of 128,256, in every way of cutting the work
  (whole, tail decoded, portions, mixed with reused pages), float32 and bfloat16, against the plain
  implementation: the head product at N = 128,256 through the engine, the fused gate/up epilogue over several
  layers, rows gathered from a mixed batch.
* 8 layers and all 32: the bfloat16 engine against the float32 engine on one 256-token prompt with the same
  (bfloat16-representable) weights.  That is a cross-check of depth, not an oracle: both sides are this
  package's kernels; what it shows is that bfloat16 rounding adds up over depth like a random walk and does
  not compound.
"""
import json

import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu

DEEP = dict(H.WIDE, vocab_size=128256, num_hidden_layers=4)


@pytest.fixture(scope="module")
def deep(tmp_path_factory):
    """The folder (weights stored in bfloat16, so both run dtypes see the same values), the requests and the
    plain implementation's logits for them, made once."""
    folder = H.make_folder(tmp_path_factory.mktemp("deep"), DEEP, 8, dtype=torch.bfloat16, std=0.02, norm_std=0.1)
    reqs = {"d0": H.random_tokens(96, DEEP["vocab_size"], 1), "d1": H.random_tokens(40, DEEP["vocab_size"], 2),
            "d2": H.random_tokens(70, DEEP["vocab_size"], 3)}
    cfg, w = P.read_model_folder(folder)
    ref = {rid: P.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    del w
    return folder, reqs, ref


def _check(got, reqs, ref, dtype):
    assert set(got) == {(rid, p) for rid, toks in reqs.items() for p in range(len(toks))}
    worst = max(float(np.abs(got[(rid, p)].astype(np.float64) - ref[rid][p]).max() / np.abs(ref[rid]).max())
                for rid, toks in reqs.items() for p in range(len(toks)))
    assert worst <= H.TOL[dtype], worst
    # the wanted rows' arg max is the plain implementation's wherever its margin is clear
    for rid, toks in reqs.items():
        for p in range(len(toks)):
            top2 = np.sort(ref[rid][p])[-2:]
            if top2[1] - top2[0] > 2 * H.TOL[dtype] * np.abs(ref[rid]).max():
                assert int(np.argmax(got[(rid, p)])) == int(np.argmax(ref[rid][p])), (rid, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_layers_at_8b_sizes_with_the_full_vocabulary(deep, dtype):
    from batchspec_b200.engine import Engine
    folder, reqs, ref = deep
    eng = Engine(dtype=dtype, device="cuda:0")
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=3, page_size=16, num_pages=16)
    for rid, sched in (("d0", H.whole("d0", reqs["d0"])), ("d1", H.tail_decoded("d1", reqs["d1"], tail=8)),
                       ("d2", H.portions("d2", reqs["d2"], [33, 2, 17, 5, 13]))):
        _check(H.run_steps_in_process(eng, sched), {rid: reqs[rid]}, ref, dtype)
    steps = H.mixed(reqs, seed=4, max_live=3, sizes=(40, 1, 2, 17, 1, 9, 1, 1))
    pages = H.max_live_tokens(steps, 16) // 16
    eng.setup_caches(max_batch_size=3, page_size=16, num_pages=pages)
    _check(H.run_steps_in_process(eng, steps), reqs, ref, dtype)
    assert eng.cache.groups[0].pool.high_water <= pages


@pytest.mark.parametrize("layers", [8, 32])
def test_depth_bfloat16_against_float32(layers):
    """The largest difference between the two run dtypes' logits, relative to the largest logit, at 8 and at all
    32 layers.  Rounding errors of separate layers add like a random walk, so the bound is the bfloat16 tolerance
    of the comparisons with the oracle (made at 1 to 4 layers) times sqrt(layers / 4); an error that a layer
    adds systematically, or one that compounds, grows faster than that and fails at 32."""
    import dataclasses
    from batchspec_b200.config import get_config
    from batchspec_b200.engine import Engine, StepEntry
    cfg = dataclasses.replace(get_config("llama-3-8b"), num_hidden_layers=layers)
    prompt = H.random_tokens(256, cfg.vocab_size, 17)
    logits = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(dtype=dtype, device="cuda:0")
        eng.load_model(config=cfg, random_seed=5, draw_on_device=True, stored_dtype=torch.bfloat16)
        eng.setup_caches(max_batch_size=1, page_size=16, num_pages=20)
        eng.admit("p")
        # most of the prompt as one portion, the rest in two more (the second crosses a page edge), then compare
        # the rows of the last portion
        eng.step([StepEntry("p", prompt[:200], ())])
        eng.step([StepEntry("p", prompt[200:231], ())])
        logits[dtype] = eng.step([StepEntry("p", prompt[231:], tuple(range(25)))]).cpu().numpy()
        del eng
        torch.cuda.empty_cache()
    ref, got = logits["float32"].astype(np.float64), logits["bfloat16"].astype(np.float64)
    assert np.isfinite(ref).all() and np.isfinite(got).all() and np.abs(ref).max() > 0.1
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err <= H.TOL["bfloat16"] * (layers / 4) ** 0.5, err
