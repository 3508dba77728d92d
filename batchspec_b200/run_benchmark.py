"""Throughput over a list of prompt lengths, in the manner of the reference's
``python -m batchspec.run_benchmark`` (batchspec/run_benchmark.py:13-100): for
every length a fresh cache sizing, ``num_total_runs`` generations of a full batch,
the first one warm-up; with ``--profiling`` each decode step is timed with CUDA
events and a report is written per length."""
from __future__ import annotations

import sys

from .args import parse_benchmark_args
from .engine import Engine
from .profiler import Profiler, register_active_profiler, release_active_profiler
from .run_e2e import load_tokenizer, setup_seed
from .runner import Runner


def main(argv=None) -> int:
    args = parse_benchmark_args(argv)
    setup_seed(args.seed)
    tokenizer = load_tokenizer(args.tokenizer_path)
    engine = Engine(tokenizer=tokenizer, dtype=args.dtype, device=args.device)
    runner = Runner(args, engine, tokenizer)
    loaded = False
    for prefix_len in args.prefix_len_list:
        args.max_len = prefix_len + args.max_gen_len
        if not loaded:
            runner.setup(max_len=args.max_len)
            loaded = True
        else:
            engine.setup_caches(max_batch_size=args.batch_size, max_seq_length=args.max_len,
                                page_size=args.page_size, prefill_chunk_size=engine.prefill_chunk_size,
                                num_pages=args.num_pages, max_tokens_per_step=engine.max_tokens_per_step)
        prof = None
        if args.profiling:
            prof = Profiler(runner_args=args)
            prof.run_name = (args.prof_run_name or "bench") + f"-bsz{args.batch_size}-prefix{prefix_len}-gen{args.max_gen_len}"
            register_active_profiler(prof)
        runner.run_benchmark(prefix_len)
        if prof is not None:
            prof.end_run()
            print(f"profiler report in {prof.save_all()}: {prof.summary['throughput_tok_s']:.1f} tok/s over timed steps")
            release_active_profiler()
    return 0


if __name__ == "__main__":
    sys.exit(main())
