"""Workload driver between the command line and the engine (the reference's
``Runner``, batchspec/runner/runner.py:21-160): ``setup`` loads the model, sizes
the caches and sets the sampling parameters; ``run_e2e`` generates for every
prompt with continuous batching; ``run_benchmark`` repeats a fixed batch
``num_total_runs`` times and reports decode throughput.

Prompts are seeded uniform token ids (``synthetic``) or lists of ids read from a
JSON / JSONL file; the reference's dataset loaders and tokenised benchmark
prefixes (runner/dataset_utils.py, runner/batch_sampler.py) are replaced by these.
"""
from __future__ import annotations

import json
import random
import time
from pathlib import Path
from typing import List, Optional

import torch

from ..engine import Engine, Sequence
from ..engine.tracer import SchedulerTracer
from ..profiler import get_active_profiler

# longest prompt portion per request and step, by batch size (runner.py:69-72)
PREFILL_CHUNK_BY_BATCH = {2: 128, 4: 128, 8: 128, 16: 128, 32: 128, 64: 64, 128: 16, 256: 8}


def synthetic_prompts(n: int, length: int, vocab: int, seed: int) -> List[List[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(length)] for _ in range(n)]


def load_prompts(path) -> List[List[int]]:
    text = Path(path).read_text().strip()
    if text.startswith("["):
        data = json.loads(text)
    else:
        data = [json.loads(line) for line in text.splitlines() if line.strip()]
    out = []
    for item in data:
        ids = item["input_ids"] if isinstance(item, dict) else item
        out.append([int(t) for t in ids])
    return out


class Runner:
    def __init__(self, args, engine: Engine, tokenizer=None):
        self.args, self.engine, self.tokenizer = args, engine, tokenizer

    def setup(self, max_len: Optional[int] = None) -> None:
        a = self.args
        if a.random_weights:
            self.engine.load_model(config_name=a.model_name, random_seed=a.seed, draw_on_device=True)
        else:
            self.engine.load_model(model_dir=a.checkpoint_path)
        max_len = max_len or a.max_len
        chunk = a.prefill_chunk or PREFILL_CHUNK_BY_BATCH.get(a.batch_size, 128)
        self.engine.setup_caches(max_batch_size=a.batch_size, max_seq_length=max_len, page_size=a.page_size,
                                 prefill_chunk_size=chunk, num_pages=a.num_pages,
                                 max_tokens_per_step=a.max_tokens_per_step or chunk * a.batch_size)
        self.engine.setup_sampling_params(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                                          force_budget=a.force_budget, seed=a.seed)
        self.engine.setup_special_tokens()
        if a.trace:
            self.engine.tracer = SchedulerTracer()

    def _prompts(self, n: int, length: int, seed: int) -> List[List[int]]:
        a = self.args
        if a.dataset == "synthetic":
            return synthetic_prompts(n, length, self.engine.config.vocab_size, seed)
        return load_prompts(a.dataset)[:n] if n else load_prompts(a.dataset)

    def run_e2e(self) -> List[Sequence]:
        a = self.args
        n = a.num_prompts or a.batch_size
        rng = random.Random(a.seed + 1)
        if a.dataset == "synthetic" and a.prefix_len_range:
            lo, hi = a.prefix_len_range
            vocab = self.engine.config.vocab_size
            prompts = [[rng.randrange(vocab) for _ in range(rng.randint(lo, hi))] for _ in range(n)]
        else:
            prompts = self._prompts(n, a.prefix_len, a.seed)
        budgets = [rng.randint(*a.gen_len_range) if a.gen_len_range else a.max_gen_len for _ in prompts]
        seqs = [Sequence(seq_id=i, prompt_ids=p, max_new_tokens=b) for i, (p, b) in enumerate(zip(prompts, budgets))]
        prof = get_active_profiler()
        prof.begin_run()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        done = self.engine.generate(seqs)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        prof.end_run()
        st = self.engine.last_stats
        if a.printoutput:
            self._print_output(done)
        print(f"Total generated tokens: {st['generated']}")
        print(f"Total model steps: {st['steps']} (batch_size: {a.batch_size}, preemptions: {st['preemptions']})")
        print(f"Mean generated tokens per step: {st['generated'] / max(st['steps'], 1):.2f}")
        print(f"Wall time: {dt:.3f} s  ({st['generated'] / dt:.1f} generated tok/s, prompts included; "
              f"{(st['generated'] + st['tokens_fed']) / dt:.1f} processed tok/s)")
        if st["decode_steps"]:
            print(f"Pure decode steps: {st['decode_steps']} of {st['steps']}, mean "
                  f"{1e3 * st['decode_seconds'] / st['decode_steps']:.2f} ms wall, "
                  f"{st['decode_tokens'] / st['decode_seconds']:.1f} tok/s over them")
        ms = sorted(st["step_ms"])
        if ms:
            pct = lambda q: ms[min(len(ms) - 1, int(q * len(ms)))]
            print(f"Step wall time ms: p50 {pct(0.5):.2f}  p90 {pct(0.9):.2f}  p99 {pct(0.99):.2f}  max {ms[-1]:.2f}")
        print("Pages: " + ", ".join(f"group {i}: high water {g.pool.high_water} of {g.pool.num_pages}"
                                    for i, g in enumerate(self.engine.cache.groups)))
        return done

    def run_benchmark(self, prefix_len: int) -> dict:
        """``num_total_runs`` generations of a full batch of ``prefix_len``-token
        prompts; decode steps are timed by the profiler, prompt steps are not part
        of the reported decode throughput."""
        a = self.args
        prof = get_active_profiler()
        gen_total = 0
        t_total = 0.0
        for run in range(a.num_total_runs):
            prompts = self._prompts(a.batch_size, prefix_len, a.seed + run)
            seqs = [Sequence(seq_id=i, prompt_ids=p, max_new_tokens=a.max_gen_len) for i, p in enumerate(prompts)]
            prof.begin_run()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            self.engine.generate(seqs)
            torch.cuda.synchronize()
            if run > 0:
                t_total += time.perf_counter() - t0
                gen_total += self.engine.last_stats["generated"]
        out = dict(prefix_len=prefix_len, batch_size=a.batch_size, runs=a.num_total_runs,
                   generated_tok_s_wall=gen_total / t_total if t_total > 0 else 0.0)
        print(f"prefix {prefix_len}: {out['generated_tok_s_wall']:.1f} generated tok/s (wall, prompts included)")
        return out

    def _print_output(self, done: List[Sequence]) -> None:
        for s in sorted(done, key=lambda s: s.seq_id):
            print(f"--- sequence {s.seq_id}: {s.status.value} ({s.finish_reason}), prompt {s.prompt_len} tokens, "
                  f"{len(s.output_ids)} generated")
            if self.tokenizer is not None:
                print(self.tokenizer.decode(s.output_ids))
            else:
                print(" ".join(str(t) for t in s.output_ids))
