"""Times single kernels of this package at the sizes of a model configuration.

    python -m batchspec_b200.kernels.microbench [--config llama-3-8b] [--what gemm attention small] [--m 1 8 64 2048]

CUDA events around each launch, after warm-up, with a read of a buffer four times
the L2 between timed launches, median of the repeats.  Prints, per kernel
and size, the time, the bytes it has to move (or the flops) and the fraction of
the peak (``MEASURED_PEAKS.json`` at the repository root if present, else the
stated fallback).
"""
from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path
from types import SimpleNamespace

import torch

from ..config import get_config
from . import ops

FALLBACK = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    out = dict(FALLBACK, source="fallback")
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            for k in FALLBACK:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
        except Exception:
            pass
    return out


class Timer:
    def __init__(self, device, flush_mb=512):
        # reading a buffer four times the L2 evicts what the last launch left without filling the L2 with dirty lines
        self.flush = torch.zeros(flush_mb << 18, dtype=torch.float32, device=device)

    def time(self, fn, warmup=3, iters=10) -> float:
        """Median milliseconds of ``fn()`` with a cold L2."""
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            self.flush.sum()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            ts.append(s.elapsed_time(e))
        return statistics.median(ts)

    def time_in_a_row(self, fn, reps: int, warmup=5, rounds=5) -> float:
        """Median milliseconds per call when ``reps`` calls follow each other without a gap (no flush of the L2
        between them: right for a kernel whose inputs the kernel before it has just written, and for kernels
        whose inputs exceed the L2 anyway)."""
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(rounds):
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(reps):
                fn()
            e.record()
            e.synchronize()
            ts.append(s.elapsed_time(e) / reps)
        return statistics.median(ts)


def bench_gemms(cfg, ms, timer, pk, dev, only=None):
    d, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    shapes = [("qkv", q + 2 * kv, d), ("o", d, q), ("gate_up", 2 * I, d), ("down", d, I), ("lm_head", V, d)]
    print(f"{'gemm':8s} {'M':>5s} {'N':>7s} {'K':>6s} | {'tcgen05 ms':>10s} {'GB/s':>7s} {'TF/s':>7s} | {'library ms':>10s} {'GB/s':>7s} {'TF/s':>7s} | frac(tc) of {pk['source']} peak")
    for name, N, K in shapes:
        if only and name not in only:
            continue
        w = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        for M in ms:
            if name == "lm_head" and M > 256:
                continue
            x = torch.randn(M, K, device=dev).bfloat16()
            out_dtype = torch.float32 if name == "lm_head" else torch.bfloat16
            t_tc = timer.time(lambda: ops.linear(x, w, out_dtype))
            t_lib = timer.time(lambda: torch.mm(x, w.t()) if out_dtype == torch.bfloat16 else torch.mm(x, w.t(), out_dtype=out_dtype))
            ops.check_status()
            byts = 2 * (N * K + M * K) + M * N * (4 if out_dtype == torch.float32 else 2)
            flops = 2.0 * M * N * K
            gb = lambda t: byts / t / 1e6
            tf = lambda t: flops / t / 1e9
            frac = max(gb(t_tc) / pk["hbm_gbs"], tf(t_tc) / pk["bf16_tflops"])
            print(f"{name:8s} {M:5d} {N:7d} {K:6d} | {t_tc:10.4f} {gb(t_tc):7.0f} {tf(t_tc):7.1f} | {t_lib:10.4f} {gb(t_lib):7.0f} {tf(t_lib):7.1f} | {frac:.3f}")


ATTENTION_CASES = [(1, 1, 2304), (8, 1, 2304), (64, 1, 2304), (8, 1, 30000), (1, 2048, 2048), (4, 512, 4096)]


def bench_attention(cfg, timer, pk, dev, page=16, cases=None, in_a_row=False):
    Hq, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    print(f"{'attention':10s} {'batch':>5s} {'q_len':>5s} {'kv_len':>6s} | {'ms':>8s} {'GB/s':>7s} {'TF/s':>7s} | frac of {pk['source']} peak")
    for batch, q_len, kv_len in cases or ATTENTION_CASES:
        pages_per = -(-kv_len // page)
        n_pages = batch * pages_per
        cache = (torch.randn(n_pages, 2, Hkv, page, hd, device=dev) * 0.5).bfloat16()
        n = batch * q_len
        qkv = torch.randn(n, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        out = torch.empty(n, Hq * hd, device=dev, dtype=torch.bfloat16)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        ctx = SimpleNamespace(
            qo_indptr=i32([i * q_len for i in range(batch + 1)]),
            positions=i32([kv_len - q_len + j for _ in range(batch) for j in range(q_len)]),
            tok_entry=i32([b for b in range(batch) for _ in range(q_len)]), n_entries=batch, n_tokens=n,
            max_q_len=q_len, max_kv_len=kv_len, extras={"min_q_len": q_len})
        tables = SimpleNamespace(kv_indptr=i32([i * pages_per for i in range(batch + 1)]),
                                 kv_indices=torch.randperm(n_pages, device=dev).to(torch.int32), page_size=page)
        call = lambda: ops.paged_attention(qkv, out, cache, ctx, tables, Hq, Hkv, hd, hd ** -0.5, 0)
        if in_a_row:                 # as many calls as take about 10 ms
            t = timer.time_in_a_row(call, max(3, min(200, int(10.0 / max(timer.time(call, iters=3), 1e-3)))))
        else:
            t = timer.time(call)
        kv_bytes = batch * kv_len * 2 * Hkv * hd * 2
        pairs = batch * (q_len * (kv_len - q_len) + q_len * (q_len + 1) / 2)
        flops = 4.0 * pairs * Hq * hd
        frac = max(kv_bytes / t / 1e6 / pk["hbm_gbs"], flops / t / 1e9 / pk["bf16_tflops"])
        print(f"{'paged':10s} {batch:5d} {q_len:5d} {kv_len:6d} | {t:8.4f} {kv_bytes / t / 1e6:7.0f} {flops / t / 1e9:7.1f} | {frac:.3f}")


def bench_small(cfg, ms, timer, pk, dev):
    d, I = cfg.hidden_size, cfg.intermediate_size
    Hq, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    print(f"{'kernel':16s} {'rows':>5s} | {'ms':>8s} {'GB/s':>7s}")
    for M in ms:
        resid = torch.randn(M, d, device=dev)
        delta = torch.randn(M, d, device=dev).bfloat16()
        w = torch.ones(d, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, d, device=dev, dtype=torch.bfloat16)
        t = timer.time(lambda: ops.add_rmsnorm(resid, delta, w, 1e-5, out))
        print(f"{'add_rmsnorm':16s} {M:5d} | {t:8.4f} {M * d * 12 / t / 1e6:7.0f}")
        u = torch.randn(M, 2 * I, device=dev).bfloat16()
        m = torch.empty(M, I, device=dev, dtype=torch.bfloat16)
        t = timer.time(lambda: ops.silu_mul(u, m, ops.GLU_GROUP))
        print(f"{'silu_mul':16s} {M:5d} | {t:8.4f} {M * I * 6 / t / 1e6:7.0f}")
        qkv = torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev).bfloat16()
        inv = ops.rope_frequency_table(500000.0 ** (-torch.arange(hd // 2, dtype=torch.float64) * 2 / hd), dev)
        pos = torch.arange(M, device=dev, dtype=torch.int32)
        ent = torch.zeros(M, device=dev, dtype=torch.int32)
        n_pages = -(-M // 16)
        cache = torch.empty(n_pages, 2, Hkv, 16, hd, device=dev, dtype=torch.bfloat16)
        indptr = torch.tensor([0, n_pages], device=dev, dtype=torch.int32)
        idx = torch.arange(n_pages, device=dev, dtype=torch.int32)
        t = timer.time(lambda: ops.rope_kv_append(qkv, Hq, Hkv, hd, inv, hd, False, pos, ent, indptr, idx, cache, 16))
        print(f"{'rope_kv_append':16s} {M:5d} | {t:8.4f} {M * (Hq + 2 * Hkv) * hd * 2 * 2 / t / 1e6:7.0f}")
    logits = torch.randn(64, cfg.vocab_size, device=dev)
    for rows in (1, 8, 64):
        t = timer.time(lambda: ops.argmax(logits[:rows]))
        print(f"{'argmax':16s} {rows:5d} | {t:8.4f} {rows * cfg.vocab_size * 4 / t / 1e6:7.0f}")
        f = lambda v, dt: torch.full((rows,), v, device=dev, dtype=dt)
        for name, k, p in (("sample", -1, 0.0), ("sample k20", 20, 0.0), ("sample p.95", -1, 0.95), ("sample k20 p.95", 20, 0.95)):
            T, K, P, sid, ctr = f(0.6, torch.float32), f(k, torch.int32), f(p, torch.float32), f(3, torch.int64), f(0, torch.int64)
            t = timer.time(lambda: ops.sample(logits[:rows], T, K, P, sid, ctr, 1))
            print(f"{name:16s} {rows:5d} | {t:8.4f} {rows * cfg.vocab_size * 4 / t / 1e6:7.0f}")


def bench_prompt_step(cfg, layers, tokens):
    """One prompt of ``tokens`` tokens through the engine's own step function, with ``layers`` of the
    configuration's layers (random weights): the step whose kernels a launch list should show."""
    import dataclasses
    import random
    from ..engine import Engine, StepEntry
    cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    eng = Engine(dtype="bfloat16", device="cuda:0")
    eng.load_model(config=cfg, random_seed=0, draw_on_device=True)
    eng.setup_caches(max_batch_size=1, max_seq_length=tokens + 16, page_size=16)
    rng = random.Random(0)
    prompt = [rng.randrange(cfg.vocab_size) for _ in range(tokens)]
    print(f"prompt step: {tokens} tokens, {layers} layers |       ms")
    for it in range(4):
        eng.admit("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        eng.step([StepEntry("p", prompt, want=(tokens - 1,))])
        end.record()
        torch.cuda.synchronize()
        eng.release("p")
        print(f"{'first (allocations, plans)' if it == 0 else 'step':>42s} | {start.elapsed_time(end):8.3f}")
    ops.check_status()


def bench_decode_step(cfg, layers, batch, context, steps=6):
    """Decode steps of ``batch`` requests that each hold ``context`` tokens, with ``layers`` of the configuration's
    layers (random weights).  The requests' pages are handed out and their lengths set without running their
    prompts (the cache holds zeros there: the traffic is the same), so the program's first
    launches are the decode steps themselves, which is what a launch list under a profiler needs."""
    import dataclasses
    from ..engine import Engine
    cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    eng = Engine(dtype="bfloat16", device="cuda:0")
    eng.load_model(config=cfg, random_seed=0, draw_on_device=True)
    eng.setup_sampling_params(temperature=0.0)
    eng.setup_caches(max_batch_size=batch, max_seq_length=context + steps + 2, page_size=16)
    for i in range(batch):
        eng.admit(i)
        eng.cache.reserve(i, context)
        eng.cache.commit(i, context)
    session = eng.decode_session(list(range(batch)), [1 + i for i in range(batch)])
    print(f"decode step: {batch} requests of {context} tokens, {layers} layers |       ms")
    for it in range(steps):
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        session.step()
        end.record()
        torch.cuda.synchronize()
        print(f"{'first (eager, then captured)' if it == 0 else 'step':>52s} | {start.elapsed_time(end):8.3f}")
    session.close()


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="llama-3-8b")
    ap.add_argument("--what", nargs="+", default=["gemm", "attention", "small"],
                    choices=["gemm", "attention", "small", "prompt-step", "decode-step"])
    ap.add_argument("--batch", type=int, default=64, help="requests of the decode step")
    ap.add_argument("--context", type=int, default=2048, help="tokens each request of the decode step holds")
    ap.add_argument("--layers", type=int, default=4, help="layers of the prompt step or the decode step")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens of the prompt step")
    ap.add_argument("--m", nargs="+", type=int, default=[1, 8, 64, 2048])
    ap.add_argument("--gemm-only", nargs="+", choices=["qkv", "o", "gate_up", "down", "lm_head"],
                    help="time only these projections")
    ap.add_argument("--attn-case", nargs=3, type=int, action="append", metavar=("BATCH", "Q_LEN", "KV_LEN"),
                    help="attention case(s) to time instead of the built-in list")
    ap.add_argument("--in-a-row", action="store_true",
                    help="attention: time calls that follow each other without a gap instead of single calls with a cold L2")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    ops.load_library()
    cfg = get_config(a.config)
    pk = peaks()
    timer = Timer(dev)
    print(f"peaks ({pk['source']}): {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s bf16")
    with torch.inference_mode():
        if "gemm" in a.what:
            bench_gemms(cfg, a.m, timer, pk, dev, only=a.gemm_only)
        if "attention" in a.what:
            bench_attention(cfg, timer, pk, dev, cases=[tuple(c) for c in a.attn_case] if a.attn_case else None,
                            in_a_row=a.in_a_row)
        if "small" in a.what:
            bench_small(cfg, [m for m in a.m if m <= 2048], timer, pk, dev)
    if "prompt-step" in a.what:
        bench_prompt_step(cfg, a.layers, a.tokens)
    if "decode-step" in a.what:
        bench_decode_step(cfg, a.layers, a.batch, a.context)


if __name__ == "__main__":
    main()
