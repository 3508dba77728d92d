"""Command-line options, grouped in dataclasses as in the reference
(batchspec/args.py:19-219) and merged into one namespace (args.py:226-301).
Option names and meanings are the reference's where it has them; its
speculative-decoding, LoRA and tensor-parallel groups are not part of this
engine.  Parsing is plain ``argparse`` built from the dataclass fields.

Reference options kept: model_name, checkpoint_path, tokenizer_path, backend,
dataset, batch_size, max_gen_len, dtype, seed, compile (accepted, ignored: the
engine has no tracing compiler), printoutput, prefix_len, prefix_len_list,
num_questions_in_prompt (accepted, synthetic prompts ignore it), num_total_runs,
temperature, top_p, top_k, force_budget, and the profiler switches.
Added: random_weights, page_size, num_pages, max_tokens_per_step, prefill_chunk,
num_prompts, trace.
"""
from __future__ import annotations

import argparse
from dataclasses import MISSING, dataclass, field, fields
from types import SimpleNamespace
from typing import List, Optional


def _str2bool(v: str) -> bool:
    if v.lower() in ("1", "true", "yes", "y", "t"):
        return True
    if v.lower() in ("0", "false", "no", "n", "f"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean, got {v!r}")


@dataclass
class CommonArguments:
    model_name: str = field(default="", metadata={"help": "Name in the by-name configuration table (used with --random_weights) and label of the run."})
    checkpoint_path: Optional[str] = field(default=None, metadata={"help": "Model folder: config.json + model.safetensors (or a sharded index)."})
    tokenizer_path: Optional[str] = field(default=None, metadata={"help": "Tokenizer folder; optional, only used to print text."})
    backend: str = field(default="standard", metadata={"help": "Backend name; this engine has 'standard' only.", "choices": ["standard"]})
    dataset: str = field(default="synthetic", metadata={"help": "'synthetic' (seeded uniform token ids) or a JSON/JSONL file of token-id lists."})
    batch_size: int = field(default=16, metadata={"help": "Most requests live at a time."})
    max_gen_len: int = field(default=128, metadata={"help": "Maximum number of tokens to generate per request."})
    dtype: str = field(default="bfloat16", metadata={"help": "bfloat16 or float32.", "choices": ["bfloat16", "float32"]})
    seed: int = field(default=42, metadata={"help": "Seed of sampling, synthetic prompts and random weights."})
    compile: bool = field(default=False, metadata={"help": "Accepted for compatibility; ignored."})
    printoutput: bool = field(default=False, metadata={"help": "Print the generated ids (and text, with a tokenizer) of each sequence."})
    random_weights: bool = field(default=False, metadata={"help": "Draw weights from --seed for the configuration --model_name instead of reading a folder."})
    page_size: int = field(default=16, metadata={"help": "Tokens per cache page."})
    num_pages: Optional[int] = field(default=None, metadata={"help": "Pages in the pool (default: batch_size x ceil(max_len / page_size))."})
    max_tokens_per_step: Optional[int] = field(default=None, metadata={"help": "Token budget of one step (default: prefill_chunk * batch_size: every request of a full batch advances one portion per step, as in the reference)."})
    prefill_chunk: Optional[int] = field(default=None, metadata={"help": "Longest prompt portion per request per step (default: by batch size, as the reference)."})
    trace: bool = field(default=False, metadata={"help": "Print the scheduler's plan and updates every step."})


@dataclass
class BenchmarkArguments:
    prefix_len_list: List[int] = field(default_factory=lambda: [1024, 2048, 4096, 8192, 12288, 16384, 20480, 24576, 28672],
                                       metadata={"help": "List of prompt lengths."})
    num_total_runs: int = field(default=11, metadata={"help": "Runs per prompt length; the first is warm-up."})


@dataclass
class E2EArguments:
    prefix_len: int = field(default=2048, metadata={"help": "Prompt length (synthetic prompts)."})
    num_questions_in_prompt: int = field(default=1, metadata={"help": "Accepted for compatibility; synthetic prompts ignore it."})
    num_total_runs: int = field(default=11, metadata={"help": "Accepted for compatibility."})
    num_prompts: Optional[int] = field(default=None, metadata={"help": "How many synthetic prompts (default: batch_size)."})
    prefix_len_range: List[int] = field(default_factory=list, metadata={"help": "LO HI: synthetic prompt lengths uniform in [LO, HI] instead of --prefix_len."})
    gen_len_range: List[int] = field(default_factory=list, metadata={"help": "LO HI: per-request token budgets uniform in [LO, HI] instead of --max_gen_len."})


@dataclass
class SamplingArguments:
    temperature: float = field(default=0.6, metadata={"help": "Temperature; 0 means greedy decoding."})
    top_p: float = field(default=0.95, metadata={"help": "Top-p (nucleus) sampling; <= 0 switches it off."})
    top_k: int = field(default=20, metadata={"help": "Top-k sampling; <= 0 switches it off."})
    force_budget: bool = field(default=False, metadata={"help": "Generate until max_gen_len is exhausted, ignoring EOS."})


@dataclass
class ProfilerArguments:
    profiling: bool = field(default=False, metadata={"help": "Time every step with CUDA events and write a report."})
    model_profiling: bool = field(default=True, metadata={"help": "Also time the kernels by bucket (embed, norm, attention, ...)."})
    engine_profiling: bool = field(default=True, metadata={"help": "Also time the host phases of a step (plan, pack, sample)."})
    prof_output_dir: str = field(default="profiler_out", metadata={"help": "Folder of the reports."})
    prof_run_name: Optional[str] = field(default=None, metadata={"help": "Name of the run's sub-folder."})
    prof_warmup_runs: int = field(default=1, metadata={"help": "Runs left out of the statistics."})
    prof_strict_sync: bool = field(default=True, metadata={"help": "Synchronise the device at step boundaries."})
    prof_kv_bins: List[int] = field(default_factory=lambda: [0, 512, 1024, 2048, 4096, 8192, 16384],
                                    metadata={"help": "Edges of the cache-length bins of the report."})
    prof_kv_len_reduce: str = field(default="mean", metadata={"help": "How a step's cache lengths become one number.",
                                                              "choices": ["mean", "max", "p50", "p90", "sum"]})


def _add_group(parser: argparse.ArgumentParser, cls) -> None:
    for f in fields(cls):
        default = f.default if f.default is not MISSING else f.default_factory()
        kw = dict(help=f.metadata.get("help", ""), default=default)
        if "choices" in f.metadata:
            kw["choices"] = f.metadata["choices"]
        t = str(f.type)
        if "bool" in t:
            parser.add_argument(f"--{f.name}", type=_str2bool, nargs="?", const=True, **kw)
        elif "List[int]" in t:
            parser.add_argument(f"--{f.name}", type=int, nargs="+", **kw)
        elif "int" in t:
            parser.add_argument(f"--{f.name}", type=int, **kw)
        elif "float" in t:
            parser.add_argument(f"--{f.name}", type=float, **kw)
        else:
            parser.add_argument(f"--{f.name}", type=str, **kw)


def _parse(groups, argv=None, prog=None) -> SimpleNamespace:
    parser = argparse.ArgumentParser(prog=prog, formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    for g in groups:
        _add_group(parser, g)
    ns = parser.parse_args(argv)
    args = SimpleNamespace(**vars(ns))
    if not args.checkpoint_path and not args.random_weights:
        parser.error("give --checkpoint_path (a model folder) or --random_weights with --model_name")
    if args.random_weights and not args.model_name:
        parser.error("--random_weights needs --model_name (a name of the configuration table)")
    args.device = "cuda:0"
    return args


def parse_benchmark_args(argv=None) -> SimpleNamespace:
    return _parse((CommonArguments, BenchmarkArguments, SamplingArguments, ProfilerArguments), argv,
                  "batchspec_b200.run_benchmark")


def parse_e2e_args(argv=None) -> SimpleNamespace:
    args = _parse((CommonArguments, E2EArguments, SamplingArguments, ProfilerArguments), argv,
                  "batchspec_b200.run_e2e")
    longest_prompt = args.prefix_len_range[1] if args.prefix_len_range else args.prefix_len
    longest_gen = args.gen_len_range[1] if args.gen_len_range else args.max_gen_len
    args.max_len = longest_prompt + longest_gen                # args.py:299 of the reference: prefix_len + max_gen_len
    return args
