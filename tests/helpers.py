"""Shared pieces of the tests: the two tiny configurations, model folders in
temporary places, replay schedules, and the comparison rule."""
from __future__ import annotations

import json
import random
from pathlib import Path

import numpy as np
import torch

import plain_llama as P

# Two tiny configurations that differ in every size and option.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=512, hidden_size=64,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176,
    rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None, max_position_embeddings=128,
    tie_word_embeddings=False)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=1000, hidden_size=96,
    num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256,
    rms_norm_eps=1e-6, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    max_position_embeddings=256, tie_word_embeddings=True)
# A third one with a larger head, more groups and odd sizes, for the kernels' other paths.
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=777, hidden_size=160,
    num_hidden_layers=2, num_attention_heads=8, num_key_value_heads=2, head_dim=64, intermediate_size=208,
    rms_norm_eps=3e-6, rope_theta=50000.0, rope_scaling=dict(rope_type="linear", factor=2.0),
    max_position_embeddings=512, tie_word_embeddings=False)
# One layer with the layer sizes of Llama-3-8B (the vocabulary cut down so that the oracle stays fast): the sizes
# at which the tensor-core kernels, and not their generic fallbacks, run.
WIDE = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", vocab_size=2048, hidden_size=4096,
    num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
    rms_norm_eps=1e-5, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    max_position_embeddings=8192, tie_word_embeddings=False)
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16)}     # config, seed, page size


def make_folder(tmp_path, cfg_json, seed, dtype=torch.float32, std=0.08, norm_std=0.1) -> Path:
    """Write a random model folder.  The spread is larger than a trained model's
    initialisation so that attention and the feed-forward move the logits."""
    from batchspec_b200.config import config_from_json_dict
    from batchspec_b200.weights import write_random_model
    return write_random_model(config_from_json_dict(cfg_json), Path(tmp_path), seed, dtype=dtype, std=std,
                              norm_std=norm_std)


def random_tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ---- tolerances, fixed before any run: largest error relative to the largest reference logit
TOL = {"float32": 2e-4, "bfloat16": 3e-2}


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    return float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max() / max(np.abs(ref).max(), 1e-30))


def oracle_logits(folder, tokens) -> np.ndarray:
    cfg, w = P.read_model_folder(folder)
    return P.forward(cfg, w, tokens).numpy()


# ---- schedules: lists of steps in trace_run's JSON form

def whole(rid, tokens, step0=0):
    return [dict(step=step0, entries=[dict(id=rid, tokens=list(tokens), want=list(range(len(tokens))))], end=[rid])]


def tail_decoded(rid, tokens, tail=32, step0=0):
    """Most of the request in one step, its last ``tail`` tokens one by one."""
    n = len(tokens)
    head = max(1, n - tail)
    steps = [dict(step=step0, entries=[dict(id=rid, tokens=list(tokens[:head]), want=list(range(head)))], end=[])]
    for i in range(head, n):
        steps.append(dict(step=step0 + len(steps), entries=[dict(id=rid, tokens=[tokens[i]], want=[0])], end=[]))
    steps[-1]["end"] = [rid]
    return steps


def portions(rid, tokens, sizes, step0=0):
    """Portions of changing size (the list of sizes is cycled)."""
    steps, pos, k = [], 0, 0
    while pos < len(tokens):
        n = min(sizes[k % len(sizes)], len(tokens) - pos)
        steps.append(dict(step=step0 + len(steps),
                          entries=[dict(id=rid, tokens=list(tokens[pos:pos + n]), want=list(range(n)))], end=[]))
        pos += n
        k += 1
    steps[-1]["end"] = [rid]
    return steps


def mixed(requests, seed, max_live=4, sizes=(5, 2, 9, 1, 3, 16, 1, 1, 7, 2)):
    """Up to ``max_live`` requests at a time; every step takes a portion (or a
    single token) of some of the live ones; a finished request ends and the next
    one starts, so its pages are handed out again.  ``requests``: {id: tokens}."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live, steps = {}, []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [toks, 0]
        entries, ended = [], []
        chosen = [rid for rid in live if rng.random() < 0.75] or [next(iter(live))]
        for rid in chosen:
            toks, pos = live[rid]
            n = min(rng.choice(sizes), len(toks) - pos)
            entries.append(dict(id=rid, tokens=list(toks[pos:pos + n]), want=list(range(n))))
            live[rid][1] = pos + n
            if pos + n == len(toks):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        steps.append(dict(step=len(steps), entries=entries, end=ended))
    return steps


def max_live_tokens(steps, round_to=64):
    """Largest sum over live requests of their length rounded up to ``round_to``."""
    held, worst = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-v // round_to) * round_to for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def run_steps_in_process(engine, steps):
    """Drive the engine's step function as bin/trace_run does.  Returns
    {(request, position): logits row}."""
    from batchspec_b200.engine import StepEntry
    out, pos = {}, {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if not engine.cache.is_live(e["id"]):
                engine.admit(e["id"])
                pos[e["id"]] = 0
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = engine.step(entries).cpu().numpy()
        r = 0
        for e in s["entries"]:
            for w in e.get("want", []):
                out[(e["id"], pos[e["id"]] + w)] = logits[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        assert r == logits.shape[0]
        for rid in s["end"]:
            engine.release(rid)
        engine.cache.check_invariants()
    assert_unused_pages_untouched(engine)
    return out


def assert_unused_pages_untouched(engine):
    """Pages are handed out lowest id first and freed ones are used again before new ones, so the ids from a
    pool's high-water mark up were never handed out: they must still hold the zeros they were allocated with.
    A stray write of any kernel (a wrong page id, a row beyond a page) into them shows here."""
    for grp in engine.cache.groups:
        pool = grp.pool
        if getattr(grp, "pages", None) is not None and pool.high_water < pool.num_pages:
            spare = grp.pages[:, pool.high_water:pool.num_pages]
            assert not bool(spare.any()), f"a page that was never handed out was written (group of {grp.spec.policy})"


def run_trace_subprocess(folder, dtype, steps, out_dir, max_tokens, extra_args=(), env=None, timeout=900):
    """Run bin/trace_run as a child, one step per line, waiting for ``done``."""
    import subprocess
    import sys
    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra_args]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline()
            assert line.strip() == f"done {s['step']}", f"trace_run said {line!r} (exit {p.poll()})"
        p.stdin.close()
        assert p.wait(timeout=timeout) == 0
    finally:
        if p.poll() is None:
            p.kill()
    out, pos = {}, {}
    vocab = json.loads((Path(folder) / "config.json").read_text())["vocab_size"]
    for s in steps:
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        if n_want:
            data = np.fromfile(Path(out_dir) / f"{s['step']}.f32", dtype="<f4").reshape(n_want, vocab)
        r = 0
        for e in s["entries"]:
            pos.setdefault(e["id"], 0)
            for w in e.get("want", []):
                out[(e["id"], pos[e["id"]] + w)] = data[r]
                r += 1
            pos[e["id"]] += len(e["tokens"])
        for rid in s["end"]:
            pos.pop(rid, None)
    return out


def compare_with_oracle(got, folder, requests, dtype_name, expect=None):
    """Every row against the plain implementation.  ``got`` has to hold exactly the rows ``expect`` (a set of
    (request, position); default: every position of every request), so a row that never came back fails the
    comparison instead of being skipped.  Returns the worst error and where it was."""
    if expect is None:
        expect = {(rid, p) for rid, toks in requests.items() for p in range(len(toks))}
    assert set(got) == set(expect), (f"{len(set(expect) - set(got))} rows missing, {len(set(got) - set(expect))} "
                                     f"unexpected, e.g. {sorted(set(expect) ^ set(got), key=str)[:4]}")
    worst = (0.0, None)
    for rid, toks in requests.items():
        ref = oracle_logits(folder, toks)
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            if (rid, p) not in expect:
                continue
            err = float(np.abs(got[(rid, p)].astype(np.float64) - ref[p]).max() / scale)
            if err > worst[0]:
                worst = (err, (rid, p))
    assert worst[0] <= TOL[dtype_name], f"worst relative error {worst[0]:.3e} at (request, position) {worst[1]}"
    return worst
