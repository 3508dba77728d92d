"""Step and bucket timing with CUDA events, statistics, JSON + Markdown reports.

Follows the reference's profiler in shape (batchspec/profiler/core.py:190-404,
timers.py:30-95): a global "active profiler" that defaults to a null object so
call sites never branch; ``step_timing_ctx`` brackets one engine step with events
(and device syncs when ``strict_sync``); named buckets collect event pairs inside
the step and are resolved to milliseconds at its end; runs before
``warmup_runs`` are left out; ``end_run`` computes count/mean/min/max/p50/p90/p99,
tokens per second = sum of tokens / sum of step time, per-bucket averages and
statistics per bin of cache length; ``save_all`` writes ``summary.json`` and
``report.md``.
"""
from __future__ import annotations

import contextlib
import json
import time
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

BUCKET_ORDER = ["embed", "norm", "attn.qkv_proj", "attn.rope", "attn.compute", "attn.o_proj",
                "mlp.gate_up_proj", "mlp.act", "mlp.down_proj", "lm_head", "sampling", "host.plan", "host.pack"]

_NULL_CTX = contextlib.nullcontext()


class NullProfiler:
    active = False

    def bucket(self, name):
        return _NULL_CTX

    def host_bucket(self, name):
        return _NULL_CTX

    def step_timing_ctx(self):
        return _NULL_CTX

    def begin_run(self):
        pass

    def end_run(self):
        pass

    def set_step_tokens(self, n):
        pass

    def set_step_seq_len(self, lens):
        pass


_active = NullProfiler()


def register_active_profiler(p) -> None:
    global _active
    _active = p


def release_active_profiler() -> None:
    global _active
    _active = NullProfiler()


def get_active_profiler():
    return _active


def bucket(name: str):
    """Context manager timing a group of kernel launches under ``name``; free when
    no profiler is registered."""
    return _active.bucket(name)


def _reduce(lens, how: str) -> float:
    a = np.asarray(lens, dtype=np.float64)
    if a.size == 0:
        return 0.0
    return float({"mean": a.mean, "max": a.max, "sum": a.sum, "p50": lambda: np.percentile(a, 50),
                  "p90": lambda: np.percentile(a, 90)}[how]())


def _stats(x: List[float]) -> Dict[str, float]:
    a = np.asarray(x, dtype=np.float64)
    if a.size == 0:
        return dict(count=0)
    return dict(count=int(a.size), mean=float(a.mean()), min=float(a.min()), max=float(a.max()),
                p50=float(np.percentile(a, 50)), p90=float(np.percentile(a, 90)), p99=float(np.percentile(a, 99)))


class Profiler:
    active = True

    def __init__(self, runner_args=None, warmup_runs: int = 1, strict_sync: bool = True,
                 kv_bins=(0, 512, 1024, 2048, 4096, 8192, 16384), kv_len_reduce: str = "mean",
                 model_profiling: bool = True, output_dir: str = "profiler_out", run_name: Optional[str] = None):
        a = runner_args
        self.args = a
        self.warmup_runs = getattr(a, "prof_warmup_runs", warmup_runs)
        self.strict_sync = getattr(a, "prof_strict_sync", strict_sync)
        self.kv_bins = list(getattr(a, "prof_kv_bins", kv_bins))
        self.kv_len_reduce = getattr(a, "prof_kv_len_reduce", kv_len_reduce)
        self.model_profiling = getattr(a, "model_profiling", model_profiling)
        self.output_dir = Path(getattr(a, "prof_output_dir", output_dir))
        self.run_name = getattr(a, "prof_run_name", run_name)
        self.run_idx = -1
        self.steps: List[dict] = []
        self.summary: Optional[dict] = None
        self._in_step = False
        self._events: List[tuple] = []
        self._host: Dict[str, float] = {}
        self._cur = None

    # -- collection ----------------------------------------------------------------
    def begin_run(self):
        self.run_idx += 1

    @property
    def _recording(self) -> bool:
        return self.run_idx >= self.warmup_runs

    @contextlib.contextmanager
    def bucket(self, name):
        if not (self._in_step and self.model_profiling) or torch.cuda.is_current_stream_capturing():
            yield
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        try:
            yield
        finally:
            e.record()
            self._events.append((name, s, e))

    @contextlib.contextmanager
    def host_bucket(self, name):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self._host[name] = self._host.get(name, 0.0) + (time.perf_counter() - t0) * 1e3

    @contextlib.contextmanager
    def step_timing_ctx(self):
        if self.strict_sync:
            torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self._in_step, self._events, self._host = True, [], {}
        self._cur = dict(tokens=0, kv_len=0.0)
        t0 = time.perf_counter()
        s.record()
        try:
            yield
        finally:
            e.record()
            e.synchronize()
            self._in_step = False
            rec = self._cur
            rec["ms"] = s.elapsed_time(e)
            rec["wall_ms"] = (time.perf_counter() - t0) * 1e3
            buckets: Dict[str, float] = {}
            for name, bs, be in self._events:
                buckets[name] = buckets.get(name, 0.0) + bs.elapsed_time(be)
            for name, ms in self._host.items():
                buckets[name] = buckets.get(name, 0.0) + ms
            rec["buckets"] = buckets
            if self._recording:
                self.steps.append(rec)

    def set_step_tokens(self, n: int):
        if self._cur is not None:
            self._cur["tokens"] = int(n)

    def set_step_seq_len(self, lens):
        if self._cur is not None:
            self._cur["kv_len"] = _reduce(lens, self.kv_len_reduce)

    # -- aggregation -----------------------------------------------------------------
    def end_run(self) -> dict:
        ms = [s["ms"] for s in self.steps]
        total_tokens = sum(s["tokens"] for s in self.steps)
        total_s = sum(ms) / 1e3
        names = sorted({k for s in self.steps for k in s["buckets"]},
                       key=lambda k: (BUCKET_ORDER.index(k) if k in BUCKET_ORDER else len(BUCKET_ORDER), k))
        per_bucket = {k: float(np.mean([s["buckets"].get(k, 0.0) for s in self.steps])) for k in names} if self.steps else {}
        edges = self.kv_bins + [float("inf")]
        bins = []
        for lo, hi in zip(edges[:-1], edges[1:]):
            sel = [s for s in self.steps if lo <= s["kv_len"] < hi]
            if sel:
                t = sum(s["ms"] for s in sel) / 1e3
                bins.append(dict(lo=lo, hi=None if hi == float("inf") else hi, steps=len(sel),
                                 mean_ms=float(np.mean([s["ms"] for s in sel])),
                                 throughput_tok_s=sum(s["tokens"] for s in sel) / t if t > 0 else 0.0))
        self.summary = dict(step_ms=_stats(ms), total_tokens=total_tokens,
                            throughput_tok_s=total_tokens / total_s if total_s > 0 else 0.0,
                            buckets_ms=per_bucket, kv_len_bins=bins, kv_len_reduce=self.kv_len_reduce,
                            runs=self.run_idx + 1, warmup_runs=self.warmup_runs)
        return self.summary

    def _dir(self) -> Path:
        d = self.output_dir / (self.run_name or "run")
        d.mkdir(parents=True, exist_ok=True)
        return d

    def save_all(self) -> Path:
        if self.summary is None:
            self.end_run()
        d = self._dir()
        (d / "summary.json").write_text(json.dumps(self.summary, indent=2) + "\n")
        s = self.summary
        lines = ["# Profiler report", "", f"- steps: {s['step_ms'].get('count', 0)}",
                 f"- tokens: {s['total_tokens']}", f"- throughput: {s['throughput_tok_s']:.1f} tok/s", ""]
        if s["step_ms"].get("count"):
            lines += ["| step ms | mean | min | p50 | p90 | p99 | max |", "|---|---|---|---|---|---|---|",
                      "| | " + " | ".join(f"{s['step_ms'][k]:.3f}" for k in ("mean", "min", "p50", "p90", "p99", "max")) + " |", ""]
        if s["buckets_ms"]:
            lines += ["| bucket | mean ms per step |", "|---|---|"] + [f"| {k} | {v:.3f} |" for k, v in s["buckets_ms"].items()] + [""]
        if s["kv_len_bins"]:
            lines += ["| cache length | steps | mean ms | tok/s |", "|---|---|---|---|"]
            lines += [f"| [{b['lo']}, {b['hi'] if b['hi'] is not None else 'inf'}) | {b['steps']} | {b['mean_ms']:.3f} | {b['throughput_tok_s']:.1f} |"
                      for b in s["kv_len_bins"]]
        (d / "report.md").write_text("\n".join(lines) + "\n")
        return d

    def save_config(self) -> None:
        if self.args is not None:
            cfg = {k: (str(v) if not isinstance(v, (int, float, str, bool, list, type(None))) else v)
                   for k, v in vars(self.args).items()}
            (self._dir() / "config.json").write_text(json.dumps(cfg, indent=2) + "\n")
