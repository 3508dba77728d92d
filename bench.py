#!/usr/bin/env python3
"""Headline benchmark: decode tokens per second of the Llama-3-8B-sized model
(random weights, bfloat16) on one B200, plus prefill of 2,048 tokens and decode at
batch 1 and 64, and the two workloads of the larger configurations: continuous batching
of 128 requests at Llama-3.2-3B sizes, and 8 prompts of 30,000 tokens at Llama-3.1-8B sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  Prints ONE JSON line.  The
decode steps are timed on the device with CUDA events; every request holds a
2,048-token prompt in the cache (put there by the engine's own prefill steps,
outside the timed region) and grows by one token per step.  A decode step reads
every weight once (15 GB, far beyond the 126 MB L2), so consecutive steps do not
reuse cached inputs.  ``e2e`` is the same workload through ``Engine.generate``
with host token ids in and out.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm))


def model_numbers(cfg, n_layers):
    """Bytes of weights one decode step reads, cache bytes per token, flops per token."""
    d, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer = d * (q + 2 * kv) + q * d + 2 * I * d + I * d + 2 * d
    weights = n_layers * per_layer + V * d + d                  # the head once; embedding rows are negligible
    return dict(weight_bytes=2 * weights, kv_bytes_per_token=n_layers * 2 * kv * 2,
                gemm_flops_per_token=2 * n_layers * (per_layer - 2 * d), head_flops_per_row=2 * V * d,
                attn_flops_per_pair=4 * n_layers * q)


def build_engine(layers, name="llama-3-8b"):
    import dataclasses
    import torch
    from batchspec_b200.config import get_config
    from batchspec_b200.engine import Engine
    cfg = get_config(name)
    full_layers = cfg.num_hidden_layers
    if layers and layers != full_layers:
        cfg = dataclasses.replace(cfg, num_hidden_layers=layers)
    eng = Engine(dtype="bfloat16", device="cuda:0")
    eng.load_model(config=cfg, random_seed=0, draw_on_device=True)
    eng.setup_sampling_params(temperature=0.0)
    return eng, cfg, full_layers


def prompts_for(batch, vocab, seed):
    import random
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(PROMPT_LEN)] for _ in range(batch)]


def run_decode(eng, cfg, batch, steps, warmup, page_size=16):
    """Device-timed decode: prefill the prompts through the engine, then
    ``warmup`` + ``steps`` decode steps; returns (ms per step, launches)."""
    import torch
    from batchspec_b200.engine import StepEntry
    from batchspec_b200.kernels import ops
    max_len = PROMPT_LEN + warmup + steps + 1
    eng.setup_caches(max_batch_size=batch, max_seq_length=max_len, page_size=page_size)
    prompts = prompts_for(batch, cfg.vocab_size, 1)
    last = []
    for i, p in enumerate(prompts):
        eng.admit(i)
        logits = eng.step([StepEntry(i, p, want=(len(p) - 1,))])
        last.append(int(ops.argmax(logits).cpu()[0]))
    session = eng.decode_session(list(range(batch)), last)
    for _ in range(warmup):
        session.step()
    torch.cuda.synchronize()
    l0 = session.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        session.step()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = session.launches - l0
    session.close()
    for i in range(batch):
        eng.release(i)
    return ms, launches


def run_prefill(eng, cfg, warmup=2, iters=3, page_size=16):
    import torch
    from batchspec_b200.engine import StepEntry
    eng.setup_caches(max_batch_size=1, max_seq_length=PROMPT_LEN + 16, page_size=page_size)
    p = prompts_for(1, cfg.vocab_size, 2)[0]
    times = []
    for it in range(warmup + iters):
        eng.admit("p")
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        eng.step([StepEntry("p", p, want=(PROMPT_LEN - 1,))])
        e.record()
        torch.cuda.synchronize()
        eng.release("p")
        if it >= warmup:
            times.append(s.elapsed_time(e))
    return statistics.median(times)


def pct(values, q):
    v = sorted(values)
    return v[min(len(v) - 1, int(q * len(v)))] if v else None


E2E_WARMUP_STEPS = 32


def run_e2e(eng, cfg, batch, steps, warmup, page_size=16):
    """The same decode workload through Engine.generate: host token ids in, host token ids out.  Every request
    generates ``warm + steps + 1`` tokens; the value is decode tokens per second over the LAST ``steps`` decode
    steps (wall clock of each step, its host->device metadata copy and device->host token read included).  The
    first ``warm`` = max(warmup, 32) decode steps are warm-up, as in the device-timed region: for about 100 ms
    after the prompt step (a quarter of a second of tensor-core work under the power cap) the SM clock stays near
    1.4 GHz before it returns to 1.9 GHz, and a decode step takes 4.9 ms instead of 4.0 ms meanwhile (clock trace
    by NVML); ``value_from_first_step`` includes those steps."""
    from batchspec_b200.engine import Sequence
    warm = max(warmup, E2E_WARMUP_STEPS)
    # token budget of one step = all prompts, so the requests prefill together and then decode in lockstep
    eng.setup_caches(max_batch_size=batch, max_seq_length=PROMPT_LEN + warm + steps + 2, page_size=page_size,
                     prefill_chunk_size=PROMPT_LEN, max_tokens_per_step=batch * PROMPT_LEN)
    eng.ignore_eos = True
    prompts = prompts_for(batch, cfg.vocab_size, 3)
    # before that: the same call on the same prompts, a few tokens (loads kernels, captures the decode graph)
    eng.generate([Sequence(i, p, max_new_tokens=4) for i, p in enumerate(prompts)])
    eng.time_decode_on_device = True
    eng.generate([Sequence(i, p, max_new_tokens=warm + steps + 1) for i, p in enumerate(prompts)])
    eng.time_decode_on_device = False
    st = eng.last_stats
    ms = st["decode_step_ms"]
    assert len(ms) == warm + steps, (len(ms), warm, steps)
    timed = ms[warm:]
    # the same steps by CUDA events around each of them: what the GPU took for them at the clock it had then
    # (the clock moves between 1.3 and 1.9 GHz under the power cap and the step follows it), so that what the
    # host adds can be told from what the clock did between this region and the device-timed one
    on_device = st["decode_step_device_ms"][warm:]
    return dict(value=round(batch * steps / (sum(timed) * 1e-3), 2), unit="tok/s",
                same_steps_on_device_ms=round(sum(on_device) / len(on_device), 3),
                of_same_steps_on_device=round(sum(on_device) / sum(timed), 4),
                h2d_bytes_per_step=st["decode_h2d_bytes_per_step"], d2h_bytes_per_step=st["decode_d2h_bytes_per_step"],
                decode_steps=steps, warmup_steps=warm, step_p50_ms=round(pct(timed, 0.5), 3),
                step_mean_ms=round(sum(timed) / len(timed), 3), step_max_ms=round(max(timed), 3),
                first_step_ms=round(ms[0], 3), value_from_first_step=round(batch * len(ms) / (sum(ms) * 1e-3), 2))


def run_cfg4(pk):
    """Continuous batching at Llama-3.2-3B sizes: 128 seeded requests, prompts of 64..4096 tokens, 16..1024 new
    tokens each, sampled (temperature 0.6, top-k 20, top-p 0.95), at most 64 at a time, prompts in portions of 512
    tokens beside the decoding requests, through ``Engine.generate``."""
    import random
    import torch
    from batchspec_b200.engine import Sequence
    eng, cfg, full_layers = build_engine(0, "llama-3.2-3b")
    eng.setup_caches(max_batch_size=64, max_seq_length=4096 + 1024 + 1, page_size=16, prefill_chunk_size=512,
                     max_tokens_per_step=4096)
    eng.setup_sampling_params(temperature=0.6, top_k=20, top_p=0.95, seed=4)
    eng.ignore_eos = True
    rng = random.Random(44)

    def workload(n):
        return [Sequence(i, [rng.randrange(cfg.vocab_size) for _ in range(rng.randint(64, 4096))],
                         max_new_tokens=rng.randint(16, 1024)) for i in range(n)]
    eng.generate(workload(8)[:8])                      # warm-up: kernels and the first graphs
    seqs = workload(128)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.generate(seqs)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.last_stats
    out = {"cfg4_tok_s": round(st["generated"] / dt, 1), "cfg4_processed_tok_s": round((st["generated"] + st["tokens_fed"]) / dt, 1),
           "cfg4_seconds": round(dt, 3), "cfg4_steps": st["steps"], "cfg4_step_p50_ms": round(pct(st["step_ms"], 0.5), 3),
           "cfg4_step_p90_ms": round(pct(st["step_ms"], 0.9), 3), "cfg4_step_p99_ms": round(pct(st["step_ms"], 0.99), 3),
           "cfg4_pages_high_water": st["pages_high_water"][0], "cfg4_pages": eng.cache.groups[0].pool.num_pages,
           "cfg4_preemptions": st["preemptions"], "cfg4_layers": cfg.num_hidden_layers}
    del eng
    torch.cuda.empty_cache()
    return out


def run_cfg5(pk):
    """Long context at Llama-3.1-8B sizes: 8 prompts of 30,000 tokens in portions of 4,096, then 256 decode steps,
    through ``Engine.generate``.  Reports the prompt phase as a fraction of the tensor-core peak and the decode
    step against the time its bytes (weights once, 8 caches) take at the measured memory rate."""
    import torch
    from batchspec_b200.engine import Sequence
    eng, cfg, full_layers = build_engine(0, "llama-3.1-8b")
    nums = model_numbers(cfg, cfg.num_hidden_layers)
    B, T, NEW, CHUNK = 8, 30000, 257, 4096
    eng.setup_caches(max_batch_size=B, max_seq_length=T + NEW + 1, page_size=16, prefill_chunk_size=CHUNK,
                     max_tokens_per_step=CHUNK)
    eng.ignore_eos = True
    prompts = [[(7919 * i + 104729 * j) % cfg.vocab_size for j in range(T)] for i in range(B)]
    eng.generate([Sequence(0, prompts[0][:CHUNK + 7], max_new_tokens=4)])          # warm-up
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    eng.generate([Sequence(i, p, max_new_tokens=NEW) for i, p in enumerate(prompts)])
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    st = eng.last_stats
    dec = st["decode_step_ms"]
    tail = dec[len(dec) // 4:]                               # the steps after the last prompt has joined
    prompt_ms = sum(st["step_ms"]) - sum(dec)
    flops = B * (T * nums["gemm_flops_per_token"] + nums["attn_flops_per_pair"] * T * (T + 1) / 2)
    step_bytes = nums["weight_bytes"] + B * (T + NEW / 2) * nums["kv_bytes_per_token"]
    p50 = pct(tail, 0.5)
    out = {"cfg5_seconds": round(dt, 3), "cfg5_prefill_tok_s": round(B * T / (prompt_ms * 1e-3), 1),
           "cfg5_prefill_tflops": round(flops / (prompt_ms * 1e-3) / 1e12, 1),
           "cfg5_prefill_frac": round(flops / (prompt_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
           "cfg5_decode_p50_ms": round(p50, 3), "cfg5_decode_steps": len(dec),
           "cfg5_decode_floor_ms": round(step_bytes / (pk["hbm_gbs"] * 1e9) * 1e3, 3),
           "cfg5_decode_frac": round(step_bytes / (p50 * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
           "cfg5_pages_per_request": -(-(T + NEW) // 16), "cfg5_layers": cfg.num_hidden_layers}
    del eng
    torch.cuda.empty_cache()
    return out


def reference_arm(a) -> int:
    """``--impl reference``: the unmodified reference through its own ``StandardEngine.generate`` (see
    baseline/reference_arm.py) on the same workload: batch, 2,048-token prompts, greedy decode steps.  If it cannot
    be imported or run, one line says why and the exit code is 0."""
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    cfg = json.loads((ROOT / "batchspec_b200" / "config" / "presets" / "llama-3-8b.json").read_text())
    full_layers = cfg["num_hidden_layers"]
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    try:
        from baseline import reference_arm as RA
        clocks = ClockSampler()
        clocks.start()
        try:
            r = RA.bench(cfg, a.batch, PROMPT_LEN, a.steps, a.warmup)
        finally:
            clock_rec = clocks.stop()
    except BaseException as exc:                                    # noqa: BLE001  (the line must say what happened)
        if isinstance(exc, KeyboardInterrupt):
            raise
        why = " ".join(f"{type(exc).__name__}: {exc}".split())[:400]
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    out = {
        "metric": f"decode tok/s (Llama-3-8B sizes, bf16, batch {a.batch}, {PROMPT_LEN}-token prompts)",
        "value": round(a.batch * 1000.0 / r["ms_per_step"], 2), "unit": "tok/s", "n_gpus": 1, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": round(r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "llama-3-8b", "global_batch": a.batch, "seq_len": PROMPT_LEN, "parallelism": "single",
                   "layers": cfg["num_hidden_layers"], "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": hd,
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": 16,
                   "weights": "random N(0,0.02)", "l2": "inputs_exceed_l2 (15 GB of weights per step)",
                   "prefill_chunk": r["chunk"],
                   "how": "StandardEngine.generate; CUDA events before each model call; tracer output discarded"},
        "clocks": clock_rec,
        "e2e": {"value": round(a.batch * 1000.0 / r["wall_ms_per_step"], 2), "unit": "tok/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": a.batch, "warmup_steps": r["warmup_steps"],
                "note": "generate keeps token ids on the device and reads one end-of-sequence flag per request"},
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0: all)")
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (no prefill, b1, b64, e2e)")
    ap.add_argument("--skip-workloads", action="store_true",
                    help="leave out e2e at batch 64 and the 3B / long-context workloads (about a minute)")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_arm(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)
    import torch
    pk = peaks()
    eng, cfg, full_layers = build_engine(a.layers)
    L = cfg.num_hidden_layers
    nums = model_numbers(cfg, L)
    section_clocks = {}

    def timed_section(name, fn, *args):
        """Runs one section with its own record of the clocks."""
        clocks = ClockSampler()
        clocks.start()
        try:
            return fn(*args)
        finally:
            section_clocks[name] = clocks.stop()

    ms, launches = timed_section("decode", run_decode, eng, cfg, a.batch, a.steps, a.warmup)
    clock_rec = section_clocks["decode"]
    value = a.batch * 1000.0 / ms
    mean_ctx = PROMPT_LEN + a.warmup + (a.steps + 1) / 2.0
    step_bytes = nums["weight_bytes"] + a.batch * mean_ctx * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s (Llama-3-8B sizes, bf16, batch {a.batch}, {PROMPT_LEN}-token prompts)", "value": round(value, 2),
        "unit": "tok/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": "llama-3-8b", "global_batch": a.batch, "seq_len": PROMPT_LEN, "parallelism": "single",
                   "layers": L, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "page_size": 16,
                   "weights": "random N(0,0.02)", "l2": "inputs_exceed_l2 (15 GB of weights per step)",
                   "peaks": pk["source"]},
        "gpu_launches": launches, "clocks": clock_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if not a.skip_points:
        # the prompt step right after the (light) decode section: it is bound by the tensor cores under the power
        # cap, and what ran just before it moves its clocks
        pms = timed_section("prefill", run_prefill, eng, cfg)
        flops = (PROMPT_LEN * nums["gemm_flops_per_token"] + nums["head_flops_per_row"]
                 + nums["attn_flops_per_pair"] * PROMPT_LEN * (PROMPT_LEN + 1) / 2)
        out["prefill"] = {"value": round(PROMPT_LEN / (pms * 1e-3), 1), "tokens": PROMPT_LEN, "ms": round(pms, 3),
                          "frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        out["e2e"] = timed_section("e2e", run_e2e, eng, cfg, a.batch, a.steps, a.warmup)
        out["e2e"]["of_device_timed"] = round(out["e2e"]["value"] / value, 4)
        points = {}
        for b in (1, 64):
            bms, _ = timed_section(f"decode_b{b}", run_decode, eng, cfg, b, a.steps, a.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / bms, 2)
            ctx_bytes = nums["weight_bytes"] + b * mean_ctx * nums["kv_bytes_per_token"]
            points[f"decode_b{b}_hbm_frac"] = round(ctx_bytes / (bms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            if b == 64 and not a.skip_workloads:
                e64 = timed_section("e2e_b64", run_e2e, eng, cfg, 64, a.steps, a.warmup)
                points["e2e_b64"] = e64["value"]
                points["e2e_b64_of_device_timed"] = round(e64["value"] / points["decode_b64"], 4)
        if not a.skip_workloads:
            del eng
            torch.cuda.empty_cache()
            points.update(timed_section("cfg4", run_cfg4, pk))
            points.update(timed_section("cfg5", run_cfg5, pk))
        out["points"] = points
        out["section_clocks"] = section_clocks
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
