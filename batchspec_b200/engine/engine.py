"""The engine: model + cache + step function + generation loop.

Method names follow the reference's ``StandardEngine``
(batchspec/backends/standard_engine.py:17-172, backends/base/engine.py:13-147):
``load_model`` -> ``setup_caches`` -> ``setup_sampling_params`` -> ``generate``.
What differs: the model comes from a folder with ``config.json`` and safetensors
(or random weights from a seed), the cache is a shared page pool instead of a
static range per slot, ``step`` is public and returns logits, and sampling is a
separate call.
"""
from __future__ import annotations

import time
from pathlib import Path
from typing import List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config import get_config, load_config
from ..kernels import ops
from ..models import get_model
from ..parts.base import Runtime
from ..profiler import get_active_profiler
from ..weights import load_weights, random_weights
from ..sampling import Sampler, SamplingParams
from .scheduler import Scheduler, Workload
from .sequence import Sequence, Status
from .step import StepEntry, StepRunner

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {dtype}")
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    return _DTYPES[dtype]


class Engine:
    def __init__(self, dtype="bfloat16", device="cuda:0", tokenizer=None):
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("batchspec_b200 runs on a CUDA device (sm_100a) only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; batchspec_b200 has no CPU path")
        self.tokenizer = tokenizer
        self.config = None
        self.model = None
        self.cache: Optional[CacheManager] = None
        self.runner: Optional[StepRunner] = None
        self.page_size = None
        self.max_batch_size = None
        self.max_seq_length = None
        self.decode_lookahead = True        # launch the next captured decode step before reading this one's tokens
        self.time_decode_on_device = False  # CUDA events around every captured decode step (last_stats: decode_step_device_ms)
        self._last_device_ms = None
        self._ahead = None
        self._stateful = False
        self._tok_host = None               # two pinned buffers that captured steps' tokens are copied into in turn
        self._tok_turn = 0
        self.prefill_chunk_size = 128
        self.max_tokens_per_step = 2048
        self.sampling = SamplingParams()
        self.sampler: Optional[Sampler] = None
        self.ignore_eos = False
        self.eos_token_ids = ()
        self.tracer = None
        self.last_stats = {}
        self.use_cuda_graphs = True
        self._graphs = {}

    # -- model -------------------------------------------------------------------
    def load_model(self, model_dir=None, config=None, config_name: Optional[str] = None,
                   random_seed: Optional[int] = None, draw_on_device: bool = False,
                   stored_dtype: Optional[torch.dtype] = None) -> None:
        """Either ``model_dir`` (config.json + safetensors), or a configuration
        (``config`` object or ``config_name`` of the by-name table) with
        ``random_seed`` for random weights."""
        ops.load_library()
        torch.cuda.set_device(self.device)
        runtime = Runtime(self.dtype, self.device)
        if model_dir is not None:
            self.config = load_config(model_dir)
            unread = getattr(self.config, "unread_keys", ())
            if unread:
                import warnings
                warnings.warn(f"config.json of {model_dir} has keys this engine does not read: {', '.join(unread)}")
            self.model = get_model(self.config, runtime)
            s = self.model.spec
            tensors = load_weights(model_dir, self.model.param_specs(), self.dtype, self.device,
                                   ignore_suffixes=s.ignore_suffixes, ignore_names=s.ignore_names,
                                   must_equal=s.must_equal)
        else:
            if config is None:
                if config_name is None:
                    raise ValueError("give model_dir, config or config_name")
                config = get_config(config_name)
            if random_seed is None:
                raise ValueError("a configuration without a folder needs random_seed")
            self.config = config
            self.model = get_model(config, runtime)
            tensors = random_weights(self.model.param_specs(), random_seed, self.dtype, self.device,
                                     draw_on_device=draw_on_device, stored_dtype=stored_dtype)
        self.model.bind(tensors)

    # -- cache -------------------------------------------------------------------
    def setup_caches(self, max_batch_size: int, max_seq_length: Optional[int] = None, page_size: int = 16,
                     prefill_chunk_size: int = 128, num_pages: Optional[int] = None,
                     max_tokens_per_step: Optional[int] = None) -> None:
        """``num_pages`` sizes every pool directly; else the pool holds
        ``max_batch_size`` requests of ``max_seq_length`` tokens (the reference's
        sizing rule, backends/base/engine.py:66-93, without its +1 page).  The token
        budget of a step defaults to ``prefill_chunk_size * max_batch_size``: a full
        batch advances by one portion per request and step, as the reference's
        chunked prefill does (standard_engine.py:176-214)."""
        if self.model is None:
            raise RuntimeError("load_model first")
        if num_pages is None:
            if max_seq_length is None:
                raise ValueError("give num_pages or max_seq_length")
            num_pages = max_batch_size * (-(-max_seq_length // page_size))
        self.page_size = page_size
        self.max_batch_size = int(max_batch_size)
        self.max_seq_length = max_seq_length
        self.prefill_chunk_size = int(prefill_chunk_size)
        self.max_tokens_per_step = int(max_tokens_per_step or prefill_chunk_size * max_batch_size)
        # the old pool (and the graphs that point into it) goes before the new one is made
        self._graphs = {}
        self._ahead = None
        self.cache = self.runner = None
        self.model.attach_caches([None] * len(self.model.spec.order))
        needs = self.model.cache_needs()
        # A step launched ahead may be dropped and run again; that repeats cache writes harmlessly but would
        # advance a mixer's per-request state twice, so models with state never launch ahead.
        self._stateful = any(need.state is not None for need in needs)
        if torch.device(self.device).type == "cuda":
            torch.cuda.empty_cache()
            want = CacheManager(needs, page_size, num_pages, max_batch_size, self.dtype, self.device,
                                allocate=False, scratch_page=True).page_bytes()
            free, _ = torch.cuda.mem_get_info(self.device)
            if want > free:
                raise ValueError(
                    f"the cache pools need {want / 2**30:.1f} GiB ({num_pages} pages of {page_size} tokens per pool) but "
                    f"{free / 2**30:.1f} GiB are free on {self.device}: lower max_batch_size or max_seq_length, or give num_pages")
        self.cache = CacheManager(needs, page_size, num_pages, max_batch_size, self.dtype, self.device, scratch_page=True)
        self.model.attach_caches(self.cache.layer_caches)
        self.runner = StepRunner(self.model, self.cache, self.model.spec.vocab_size, self.device)

    # -- the step function ---------------------------------------------------------
    def admit(self, req_id) -> None:
        self.cache.admit(req_id)

    def release(self, req_id) -> None:
        self.cache.release(req_id)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        return self.runner.step(entries)

    def decode_graph(self, batch: int):
        """The captured decode step for ``batch`` entries, or None when graphs are
        off or the longest request is not bounded (no ``max_seq_length``)."""
        if not self.use_cuda_graphs or not self.max_seq_length or not self.model.graph_safe:
            return None
        prof = get_active_profiler()
        if prof.active and getattr(prof, "model_profiling", False):
            return None                       # per-kernel buckets need the kernels launched one by one
        # one graph per bucket of batch sizes (1, 2, 4, 8, 16, 24, ...): smaller steps are padded with rows that
        # write to, and attend over, the cache's scratch page
        bucket = batch
        if self.cache.scratch_pages() is not None:
            bucket = 1
            while bucket < batch:
                bucket = bucket * 2 if bucket < 8 else bucket + 8
            bucket = max(batch, min(bucket, self.max_batch_size))
        if bucket not in self._graphs:
            from .decode_graph import DecodeGraph
            self._graphs[bucket] = DecodeGraph(self, bucket, self.max_seq_length)
        return self._graphs[bucket]

    def decode_session(self, req_ids, first_tokens):
        """A device-resident greedy decode loop over live requests (see DecodeSession)."""
        from .decode_session import DecodeSession
        return DecodeSession(self, req_ids, first_tokens)

    # -- sampling ------------------------------------------------------------------
    def setup_sampling_params(self, temperature: float = 0.0, top_k: int = -1, top_p: float = 0.0,
                              force_budget: bool = False, seed: int = 0) -> None:
        """Names as in the reference (backends/base/engine.py:95-113).  ``force_budget``
        keeps generating to the token budget, never stopping at EOS
        (standard_engine.py:230-232); the reference's replacement of an
        end-of-thinking token by filler words is not part of this engine."""
        self.sampling = SamplingParams(float(temperature), int(top_k), float(top_p))
        self.ignore_eos = bool(force_budget)
        self.sampler = Sampler(self.device, seed, self.sampling)

    def setup_special_tokens(self, eos_token_ids=None) -> None:
        """EOS ids: the argument, else the tokenizer's, else config.json's
        (backends/base/engine.py:116-147 takes them from the tokenizer)."""
        if eos_token_ids is not None:
            self.eos_token_ids = tuple(int(t) for t in eos_token_ids)
        elif self.tokenizer is not None and getattr(self.tokenizer, "eos_token_id", None) is not None:
            self.eos_token_ids = (int(self.tokenizer.eos_token_id),)
        else:
            self.eos_token_ids = tuple(getattr(self.config, "eos_token_ids", ()) or ())

    # -- generation ----------------------------------------------------------------
    def make_scheduler(self) -> Scheduler:
        max_len = getattr(self.config, "max_position_embeddings", None) or (1 << 30)
        if self.max_seq_length:
            max_len = min(max_len, self.max_seq_length)
        return Scheduler(self.cache, self.max_batch_size, self.max_tokens_per_step, self.prefill_chunk_size,
                         max_len, self.eos_token_ids, self.ignore_eos)

    def sample_workloads(self, workloads: List[Workload], logits: torch.Tensor) -> torch.Tensor:
        wanting = [w.seq for w in workloads if w.wants_token]
        d = self.sampling
        return self.sampler.sample(
            logits,
            [d.temperature if s.temperature is None else s.temperature for s in wanting],
            [d.top_k if s.top_k is None else s.top_k for s in wanting],
            [d.top_p if s.top_p is None else s.top_p for s in wanting],
            [s.seq_id for s in wanting], [len(s.output_ids) for s in wanting])

    def _launch_decode(self, graph, seqs, tokens, ahead: int):
        """Enqueue one captured decode step of ``seqs`` and the copy of its chosen tokens into pinned host memory.
        ``tokens`` None: the step's input ids are the ones the step before left on the device.  ``ahead``: 1 if
        the step before has not been accounted for on the host yet (its output token counts as drawn)."""
        d = self.sampling
        ids = [s.seq_id for s in seqs]
        for rid in ids:
            self.cache.reserve(rid, 1)
        timed = self.time_decode_on_device
        if timed:
            begin = torch.cuda.Event(enable_timing=True)
            begin.record()
        out = graph.run(ids, tokens,
                        [d.temperature if s.temperature is None else s.temperature for s in seqs],
                        [d.top_k if s.top_k is None else s.top_k for s in seqs],
                        [d.top_p if s.top_p is None else s.top_p for s in seqs],
                        ids, [len(s.output_ids) + ahead for s in seqs])
        k = self._tok_turn = (self._tok_turn + 1) % 2
        if self._tok_host is None or self._tok_host[0].numel() < self.max_batch_size:
            self._tok_host = [torch.empty((self.max_batch_size,), dtype=torch.int32).pin_memory() for _ in range(2)]
        host = self._tok_host[k][:len(ids)]
        host.copy_(out, non_blocking=True)
        ops.status_to_host_async()
        ev = torch.cuda.Event(enable_timing=timed)
        ev.record()
        return dict(graph=graph, ids=ids, host=host, event=ev, begin=begin if timed else None, h2d=graph.last_h2d_bytes)

    def _graph_decode_step(self, graph, work: List[Workload], sched: Optional[Scheduler] = None) -> List[int]:
        """A pure decode step through the captured graph: host token ids in, host token ids out.

        With a scheduler at hand the step AFTER this one is launched before this one's tokens are read, whenever it
        is certain to be the same requests again unless one of them ends on a token only the GPU knows yet: the
        host's work for a step (reading tokens, updating and planning, filling and uploading the next step's
        metadata, the graph launch) then overlaps with the GPU instead of alternating with it.  The step launched
        ahead takes its input ids from the device.  If the next plan turns out to be a subset of it (a request hit
        an end-of-sequence token), its tokens are used for the requests that go on; if not, it is dropped: it wrote
        keys that the real step writes again, and its page reservations are the real step's."""
        seqs = [w.seq for w in work]
        ids = [s.seq_id for s in seqs]
        cur, ahead = None, self._ahead
        self._ahead = None
        if ahead is not None and set(ids) <= set(ahead["ids"]):
            cur = ahead                                    # this step is already running (or done)
        if cur is None:
            cur = self._launch_decode(graph, seqs, [s.known_token(w.start) for s, w in zip(seqs, work)], 0)
        for rid in ids:
            self.cache.commit(rid, 1)
        # Launch the next step now?  Only when the next plan cannot differ from this one except by requests that end
        # on a token the host does not know yet: every live request is in this step (none is in the middle of its
        # prompt, held up for pages that an ending request would free), nobody waits for admission (or no slot can
        # come free: all are taken and no request stops at an end-of-sequence token), nobody reaches a length limit
        # with this step's token, and the pages the next step needs are free.
        if (sched is not None and self.decode_lookahead and not self._stateful and cur["ids"] == ids
                and cur["graph"] is graph
                and len(sched.running) == len(ids)
                and (not sched.waiting_queue or (sched.ignore_eos and len(sched.running) >= sched.max_concurrency))
                and self.tracer is None and not get_active_profiler().active
                and all(len(s.output_ids) + 1 < s.max_new_tokens and s.total_len + 1 < sched.max_model_len
                        for s in seqs)):
            need = [sum(col) for col in zip(*(self.cache.pages_missing(rid, 1) for rid in ids))]
            if all(n <= g.pool.num_free for n, g in zip(need, self.cache.groups)):
                self._ahead = self._launch_decode(graph, seqs, None, 1)
        cur["event"].synchronize()
        ops.raise_if_gave_up()
        # the step's own time on the device (its upload, kernels and the copy of its tokens), without whatever
        # the stream waited for the host before it
        self._last_device_ms = cur["begin"].elapsed_time(cur["event"]) if cur["begin"] is not None else None
        toks = cur["host"].tolist()
        self._last_h2d = cur["h2d"]
        if cur["ids"] == ids:
            return toks
        where = {rid: i for i, rid in enumerate(cur["ids"])}
        return [toks[where[rid]] for rid in ids]

    @torch.inference_mode()
    def generate(self, sequences: List[Sequence]) -> List[Sequence]:
        """Continuous batching until every sequence is finished
        (standard_engine.py:145-172): plan -> step -> sample -> update.  Token ids
        go in and come out on the host."""
        if self.sampler is None:
            self.setup_sampling_params()
        self.cache.release_all()
        self._ahead = None
        sched = self.make_scheduler()
        sched.add_sequences(sequences)
        steps = tokens_in = 0
        dec_steps = dec_tokens = dec_h2d = dec_d2h = 0
        dec_seconds = 0.0
        step_ms, dec_step_ms, dec_device_ms = [], [], []
        prof = get_active_profiler()
        while not sched.is_done():
            t_step = time.perf_counter()
            with prof.host_bucket("host.plan"):
                work = sched.plan()
            if not work:
                break
            if self.tracer is not None:
                self.tracer.on_plan(steps, sched, work)
            wanting = [w for w in work if w.wants_token]
            graph = self.decode_graph(len(work)) if len(wanting) == len(work) and all(
                w.n_tokens == 1 for w in work) else None
            with prof.step_timing_ctx():
                if graph is not None:
                    toks = self._graph_decode_step(graph, work, sched)
                    h2d = self._last_h2d
                    if self._last_device_ms is not None:
                        dec_device_ms.append(self._last_device_ms)
                else:
                    self._ahead = None        # a step launched ahead stands for the very next step or for none
                    entries = [StepEntry(w.seq.seq_id, w.seq.known_tokens(w.start, w.start + w.n_tokens),
                                         (w.n_tokens - 1,) if w.wants_token else ()) for w in work]
                    logits = self.runner.step(entries)
                    with prof.bucket("sampling"):
                        chosen = self.sample_workloads(work, logits) if wanting else None
                        ops.status_to_host_async()
                        toks = chosen.cpu().tolist() if wanting else []
                        if wanting:
                            ops.raise_if_gave_up()
                    h2d = self.runner.last_h2d_bytes
                prof.set_step_tokens(len(wanting))
                prof.set_step_seq_len([w.start + w.n_tokens for w in work])
            sched.process_results(work, {w.seq.seq_id: t for w, t in zip(wanting, toks)})
            if self.tracer is not None:
                self.tracer.on_update(steps, sched, work, toks)
            steps += 1
            step_ms.append((time.perf_counter() - t_step) * 1e3)
            tokens_in += sum(w.n_tokens for w in work)
            if len(wanting) == len(work) and all(w.n_tokens == 1 for w in work):      # a pure decode step
                dec_steps += 1
                dec_tokens += len(work)
                dec_seconds += time.perf_counter() - t_step
                dec_step_ms.append(step_ms[-1])
                dec_h2d += h2d
                dec_d2h += 4 * len(work)
        self.last_stats = dict(steps=steps, tokens_fed=tokens_in, preemptions=sched.num_preemptions,
                               generated=sum(len(s.output_ids) for s in sched.completed),
                               step_ms=step_ms, decode_step_ms=dec_step_ms, decode_step_device_ms=dec_device_ms,
                               decode_steps=dec_steps,
                               pages_high_water=[g.pool.high_water for g in self.cache.groups], decode_tokens=dec_tokens, decode_seconds=dec_seconds,
                               decode_h2d_bytes_per_step=dec_h2d // max(dec_steps, 1),
                               decode_d2h_bytes_per_step=dec_d2h // max(dec_steps, 1))
        return sched.completed
