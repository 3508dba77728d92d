"""Continuous-batching scheduler above the step function.

The reference's scheduler (batchspec/backends/continuous/scheduler.py:34-295) has a
fixed array of batch slots, admits FIFO into free slots, plans decode entries
first and then one chunk of ``prefill_chunk_len`` for every prefilling slot, and
pads empty slots with dummy tokens; pages cannot run out because each slot owns a
static range.  This one keeps the policy (FIFO admission, decode first, chunked
prompts, the PREFILL -> DECODE -> COMPLETE states, scheduler.py:251-282) and adds
what a shared page pool needs:

* a token budget per step (``max_tokens_per_step``): decode tokens first, the rest
  is dealt to prefilling requests in admission order, so portions change size from
  step to step;
* admission only while a request slot is free and the pool can hold the first
  portion;
* when pages run out for requests that are already running, the most recently
  admitted live request is preempted: its pages go back, it returns to the head
  of the waiting queue and will recompute prompt + generated tokens when it is
  admitted again.  A request that could never fit (longer than the model's
  context, or needing more pages than the whole pool) fails with a reason instead
  of running.

Finish rule: an EOS token (unless ``ignore_eos``), ``max_new_tokens`` reached, the
context is full, or ("cache") the request alone has outgrown the whole pool; tested on every generated token, the first included (the
reference skips the first, scheduler.py:255-260).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional, Sequence as Seq

from ..cache.manager import CacheManager
from .sequence import Sequence, Status


@dataclass
class Workload:
    """What one live request does in the next step."""
    seq: Sequence
    start: int            # index of the first token fed (== tokens already in the cache)
    n_tokens: int
    wants_token: bool     # True when the portion ends at the last known token


class Scheduler:
    def __init__(self, cache: CacheManager, max_concurrency: int, max_tokens_per_step: int,
                 prefill_chunk_len: int, max_model_len: int, eos_token_ids: Seq[int] = (),
                 ignore_eos: bool = False):
        if max_tokens_per_step < 1 or prefill_chunk_len < 1 or max_concurrency < 1:
            raise ValueError("max_concurrency, max_tokens_per_step and prefill_chunk_len must be >= 1")
        self.cache = cache
        self.max_concurrency = int(max_concurrency)
        self.max_tokens_per_step = int(max_tokens_per_step)
        self.prefill_chunk_len = int(prefill_chunk_len)
        self.max_model_len = int(max_model_len)
        self.eos_token_ids = frozenset(int(t) for t in eos_token_ids)
        self.ignore_eos = bool(ignore_eos)
        self.waiting_queue: Deque[Sequence] = deque()
        self.running: List[Sequence] = []          # in admission order
        self.completed: List[Sequence] = []
        self.total = 0
        self.num_preemptions = 0
        self._admissions = 0

    # -- queue ---------------------------------------------------------------------
    def add_sequences(self, sequences: Seq[Sequence]) -> None:
        for s in sequences:
            self.total += 1
            s.status = Status.PENDING
            reason = self._never_fits(s)
            if reason:
                self._finish(s, Status.FAILED, reason)
            else:
                self.waiting_queue.append(s)

    def is_done(self) -> bool:
        return len(self.completed) == self.total

    @staticmethod
    def _fits(need: List[int], free: List[int]) -> bool:
        return all(n <= f for n, f in zip(need, free))

    @staticmethod
    def _take(need: List[int], free: List[int]) -> List[int]:
        return [f - n for n, f in zip(need, free)]

    def _never_fits(self, s: Sequence) -> Optional[str]:
        if s.prompt_len < 1:
            return "empty prompt"
        if s.max_new_tokens < 1:
            return "max_new_tokens must be >= 1"
        if s.prompt_len + 1 > self.max_model_len:
            return f"prompt of {s.prompt_len} tokens does not fit the context of {self.max_model_len}"
        first = min(self.prefill_chunk_len, self.max_tokens_per_step, s.prompt_len)
        if self._outgrows_a_pool(s.prompt_len + 1) or not self._fits(
                self.cache.pages_needed(0, first), [g.pool.num_pages for g in self.cache.groups]):
            return f"prompt of {s.prompt_len} tokens needs more pages than the whole pool has"
        return None

    def _outgrows_a_pool(self, total_len: int) -> bool:
        """True if a request of this many tokens, alone in the cache and fed token by token (portions shrink to the
        room there is), would still need more pages of a group than that group's pool has.  A window's group only
        ever holds the window and the tokens in flight."""
        return any(need > g.pool.num_pages
                   for need, g in zip(self.cache.peak_pages(total_len, 1), self.cache.groups))

    # -- planning ------------------------------------------------------------------
    def _preempt_latest(self) -> Sequence:
        victim = max(self.running, key=lambda s: s.admitted_at)
        self.running.remove(victim)
        self.cache.release(victim.seq_id)
        victim.num_computed = 0
        victim.status = Status.PENDING
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting_queue.appendleft(victim)
        return victim

    def plan(self) -> List[Workload]:
        """Workloads of the next step.  May preempt; never plans more pages than
        are free, so the step's reservation cannot fail."""
        cache = self.cache
        while True:
            # a live request whose known tokens no longer fit the whole pool can never go on
            for s in [s for s in self.running if self._outgrows_a_pool(s.total_len)]:
                self._retire(s, "cache")
            budget = self.max_tokens_per_step
            free = cache.free_pages()
            work: List[Workload] = []
            starved = False
            # 1. decode entries first, in admission order
            for s in self.running:
                if s.status is not Status.DECODE:
                    continue
                need = cache.pages_missing(s.seq_id, 1)
                if budget < 1:
                    break
                if not self._fits(need, free):
                    starved = True
                    break
                free = self._take(need, free)
                budget -= 1
                work.append(Workload(s, s.num_computed, 1, True))
            # 2. portions of requests that are already prefilling
            if not starved:
                for s in self.running:
                    if s.status is not Status.PREFILL or budget < 1:
                        continue
                    n = self._portion(s, budget, free)
                    if n == 0:
                        continue
                    free = self._take(cache.pages_missing(s.seq_id, n), free)
                    budget -= n
                    work.append(Workload(s, s.num_computed, n, s.num_computed + n == s.total_len))
            # 3. admit waiting requests while slots, budget and pages allow
            if not starved:
                while (self.waiting_queue and len(self.running) < self.max_concurrency
                       and cache.slots.num_free > 0 and budget >= 1):
                    s = self.waiting_queue[0]
                    n = min(self.prefill_chunk_len, s.total_len, budget)
                    if not self._fits(cache.pages_needed(0, n), free):      # the whole first portion must fit
                        break
                    self.waiting_queue.popleft()
                    cache.admit(s.seq_id)
                    s.status = Status.PREFILL
                    s.admitted_at = self._admissions
                    self._admissions += 1
                    self.running.append(s)
                    free = self._take(cache.pages_needed(0, n), free)
                    budget -= n
                    work.append(Workload(s, 0, n, n == s.total_len))
            if work and not starved:
                return work
            if not self.running:
                if self.waiting_queue:
                    # nothing runs and the head cannot start: it can never fit
                    s = self.waiting_queue.popleft()
                    self._finish(s, Status.FAILED, "needs more pages than the pool can ever free")
                    continue
                return []
            # live requests cannot move: give the latest one's pages to the others
            self._preempt_latest()

    def _portion(self, s: Sequence, budget: int, free_pages: List[int]) -> int:
        """Largest portion of s's remaining known tokens within the chunk length,
        the step's budget and the free pages of every group."""
        remaining = s.total_len - s.num_computed
        n = min(self.prefill_chunk_len, remaining, budget)
        if n <= 0:
            return 0
        return max(0, min(n, self.cache.room_for(s.num_computed, free_pages)))

    # -- results -------------------------------------------------------------------
    def process_results(self, workloads: Seq[Workload], next_tokens: Dict[int, int]) -> None:
        """``next_tokens``: seq_id -> sampled token, for workloads with
        ``wants_token``.  The cache lengths were already advanced by the step."""
        for w in workloads:
            s = w.seq
            s.num_computed += w.n_tokens
            if not w.wants_token:
                continue
            tok = int(next_tokens[s.seq_id])
            s.output_ids.append(tok)
            s.status = Status.DECODE
            if tok in self.eos_token_ids and not self.ignore_eos:
                self._retire(s, "eos")
            elif len(s.output_ids) >= s.max_new_tokens:
                self._retire(s, "length")
            elif s.total_len >= self.max_model_len:
                self._retire(s, "context")

    def _retire(self, s: Sequence, reason: str) -> None:
        self.running.remove(s)
        self.cache.release(s.seq_id)
        self._finish(s, Status.COMPLETE, reason)

    def _finish(self, s: Sequence, status: Status, reason: str) -> None:
        s.status = status
        s.finish_reason = reason
        self.completed.append(s)
