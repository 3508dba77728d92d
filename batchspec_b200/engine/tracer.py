"""Prints what the scheduler decided and what came back, step by step (the
reference's SchedulerTracer, batchspec/backends/continuous/tracer.py:29-139, which
is always on there; here it is behind ``--trace``)."""
from __future__ import annotations

import sys


class SchedulerTracer:
    def __init__(self, stream=None):
        self.stream = stream or sys.stdout

    def on_plan(self, step, sched, work):
        parts = [f"{w.seq.seq_id}:{w.seq.status.value}[{w.start}+{w.n_tokens}]{'*' if w.wants_token else ''}"
                 for w in work]
        free = [g.pool.num_free for g in sched.cache.groups]
        print(f"[step {step}] PLAN   {' '.join(parts)} | waiting={len(sched.waiting_queue)} "
              f"running={len(sched.running)} free_pages={free}", file=self.stream)

    def on_update(self, step, sched, work, tokens):
        wanting = [w for w in work if w.wants_token]
        parts = [f"{w.seq.seq_id}->{t}{'(' + w.seq.finish_reason + ')' if w.seq.finish_reason else ''}"
                 for w, t in zip(wanting, tokens)]
        print(f"[step {step}] UPDATE {' '.join(parts)} | done={len(sched.completed)}/{sched.total} "
              f"preemptions={sched.num_preemptions}", file=self.stream)
