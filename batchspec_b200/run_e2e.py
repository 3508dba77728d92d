"""End-to-end generation from the command line, in the manner of the reference's
``python -m batchspec.run_e2e`` (batchspec/run_e2e.py:14-79):

    python -m batchspec_b200.run_e2e --checkpoint_path DIR --batch_size 16 \\
        --prefix_len 256 --max_gen_len 128 --temperature 0.0 [--printoutput]
    python -m batchspec_b200.run_e2e --random_weights --model_name llama-3-8b ...
"""
from __future__ import annotations

import random
import sys

import numpy as np
import torch

from .args import parse_e2e_args
from .engine import Engine
from .profiler import Profiler, register_active_profiler, release_active_profiler
from .runner import Runner


def setup_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def load_tokenizer(path):
    if not path:
        return None
    from transformers import AutoTokenizer           # tokenizer only; no model code of that package is used
    tok = AutoTokenizer.from_pretrained(path, padding_side="right", local_files_only=True)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    return tok


def main(argv=None) -> int:
    args = parse_e2e_args(argv)
    setup_seed(args.seed)
    tokenizer = load_tokenizer(args.tokenizer_path)
    engine = Engine(tokenizer=tokenizer, dtype=args.dtype, device=args.device)
    runner = Runner(args, engine, tokenizer)
    runner.setup()
    prof = None
    if args.profiling:
        prof = Profiler(runner_args=args)
        prof.warmup_runs = 0
        register_active_profiler(prof)
    runner.run_e2e()
    if prof is not None:
        prof.save_config()
        print(f"profiler report in {prof.save_all()}")
        release_active_profiler()
    return 0


if __name__ == "__main__":
    sys.exit(main())
