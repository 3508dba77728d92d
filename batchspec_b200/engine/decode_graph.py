"""Decode steps as CUDA graphs.

A step in which every entry is one token of a live request has the same kernels
and launch sizes whenever the number of entries is the same; only the metadata
(positions, block tables, state slots, sampling counters) and the token ids
differ.  ``DecodeGraph`` keeps that metadata in one device buffer with a fixed
layout, captures model forward + sampling once per batch size, and replays it
with a fresh upload per step.  The kernels read everything that changes from the
buffer, never from launch arguments.  This replaces the reference's
``torch.compile`` of the step (batchspec/backends/standard_engine.py:103-106).

Layout of the int32 metadata buffer for B entries and at most P_g pages per request in
cache group g (``dyn`` is uploaded every step, the tables only when a page was added):

    dyn:    the fields of ``step.CONTEXT_FIELDS`` for B entries of one token each, then
            top_k[B] temperature[B] (f32) top_p[B] (f32) stream_id[B] (i64) counter[B] (i64)
    const:  kv_indptr[B+1] per group
    tables: kv_indices[B * P_g] per group

The values of the context fields come from ``step.step_fields``, the same function that packs
an ordinary step; rows beyond the live requests are its padding entries.
"""
from __future__ import annotations

import gc

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .step import CONTEXT_FIELDS, GroupTables, StepContext, field_length, step_fields


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class DecodeGraph:
    def __init__(self, engine, batch: int, max_kv_len: int):
        self.engine, self.B = engine, int(batch)
        self.max_kv_len = int(max_kv_len)
        cache = engine.cache
        B, ng = self.B, len(cache.groups)
        self.P = [-(-self.max_kv_len // g.page_size) for g in cache.groups]      # table entries per row, per group
        off, o = {}, 0
        for name, kind in CONTEXT_FIELDS:
            off[name] = o
            o += _align(field_length(kind, B, B, B))
        assert off["token_ids"] == 0                  # a step whose ids are on the device uploads from the next field on
        for name in ("top_k", "temperature", "top_p"):
            off[name] = o
            o += _align(B)
        o = _align(o, 2)
        for name in ("stream_id", "counter"):
            off[name] = o
            o += _align(2 * B)
        self.dyn_len = o
        for g in range(ng):
            off[f"kv_indptr{g}"] = o
            o += _align(B + 1)
        self.table_begin = o
        for g in range(ng):
            off[f"kv_indices{g}"] = o
            o += _align(B * self.P[g])
        self.total = o
        self.off = off
        self.meta = np.zeros(self.total, dtype=np.int32)                 # the authoritative host copy
        for g in range(ng):
            self.meta[off[f"kv_indptr{g}"]:off[f"kv_indptr{g}"] + B + 1] = np.arange(B + 1) * self.P[g]
        self.ring = [torch.empty(self.total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self.ring_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self.turn = 0
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=engine.device)
        self.row_req: List[object] = [None] * B
        self.row_pages = [[0] * ng for _ in range(B)]
        self.tables_dirty = True
        self.const_uploaded = False
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.next_tokens: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self.kernels_per_replay = 0
        self.uses = 0
        self.last_h2d_bytes = 0
        d = self.dev
        view = lambda name, n: d[off[name]:off[name] + n]
        f32 = lambda name: d[off[name]:off[name] + B].view(torch.float32)
        i64 = lambda name: d[off[name]:off[name] + 2 * B].view(torch.int64)
        self.v_temperature, self.v_top_p = f32("temperature"), f32("top_p")
        self.v_top_k = view("top_k", B)
        self.v_stream, self.v_counter = i64("stream_id"), i64("counter")
        tables = [GroupTables(grp.page_size, view(f"kv_indptr{g}", B + 1), view(f"kv_indices{g}", B * self.P[g]), None, None)
                  for g, grp in enumerate(cache.groups)]
        views = {name: view(name, field_length(kind, B, B, B)) for name, kind in CONTEXT_FIELDS}
        self.v_tokens = views["token_ids"]
        self.ctx = StepContext(n_tokens=B, n_entries=B, n_logit_rows=B, tables=tables, max_q_len=1,
                               max_kv_len=self.max_kv_len, host=None, extras={"min_q_len": 1, "captured": True}, **views)

    # -- host side -------------------------------------------------------------------
    _PAD = object()        # marks a table row that currently points at the scratch page

    def _fill(self, req_ids: Sequence, tokens: Optional[Sequence[int]], temperature, top_k, top_p, stream_ids,
              counters) -> None:
        cache, off, B, m = self.engine.cache, self.off, self.B, self.meta
        n = len(req_ids)
        reqs = [cache.requests[r] for r in req_ids]
        # rows n .. B-1 are padding: one token at position 0 of the scratch page and the scratch state slot,
        # greedy, result ignored
        fields, _ = step_fields(cache, list(req_ids) + [None] * (B - n), [1] * B, [(0,)] * B,
                                None if tokens is None else [[t] for t in tokens] + [[0]] * (B - n), with_tables=False)
        for name, _kind in CONTEXT_FIELDS:
            if name == "token_ids" and tokens is None:
                continue
            v = fields[name]
            m[off[name]:off[name] + v.shape[0]] = v

        def put(name, values, view=None, width=1):
            dst = m[off[name]:off[name] + width * B]
            if view is not None:
                dst = dst.view(view)
            dst[:n] = values
            dst[n:] = 0

        put("top_k", top_k)
        put("temperature", temperature, np.float32)
        put("top_p", top_p, np.float32)
        put("stream_id", stream_ids, np.int64, 2)
        put("counter", counters, np.int64, 2)
        if n < B:
            scratch = cache.scratch_pages()
            for i in range(n, B):
                if self.row_req[i] is not self._PAD:
                    for g, page in enumerate(scratch):
                        m[off[f"kv_indices{g}"] + i * self.P[g]] = page
                        self.row_pages[i][g] = 0
                    self.row_req[i] = self._PAD
                    self.tables_dirty = True
        for i, (rid, rc) in enumerate(zip(req_ids, reqs)):
            # the row's table on the device is this request's only if it is the same admission: a request that was
            # preempted and admitted again has the same id but other pages (perhaps as many as before)
            fresh = self.row_req[i] != (rid, rc.serial)
            for g, table in enumerate(rc.tables):
                have = 0 if fresh else self.row_pages[i][g]
                P = self.P[g]
                if len(table) > P:
                    raise RuntimeError(f"request {rid!r} holds {len(table)} pages, the captured step allows {P}")
                if fresh or len(table) != have:
                    base = off[f"kv_indices{g}"] + i * P
                    lo = 0 if fresh or len(table) < have else have
                    m[base + lo:base + len(table)] = table[lo:]
                    self.row_pages[i][g] = len(table)
                    self.tables_dirty = True
                elif cache.groups[g].spec.policy == "window":
                    base = off[f"kv_indices{g}"] + i * P         # released pages turn into -1 in place
                    m[base:base + len(table)] = table
                    self.tables_dirty = True
            self.row_req[i] = (rid, rc.serial)

    def _upload(self, with_tokens: bool) -> None:
        i = self.turn
        self.turn = (self.turn + 1) % len(self.ring)
        if self.ring_events[i] is not None:
            self.ring_events[i].synchronize()
        host = self.ring[i]
        B = self.B
        lo = 0 if with_tokens else self.off["positions"]
        hi = self.total if (self.tables_dirty or not self.const_uploaded) else self.dyn_len
        host.numpy()[lo:hi] = self.meta[lo:hi]
        self.dev[lo:hi].copy_(host[lo:hi], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.ring_events[i] = ev
        self.tables_dirty = False
        self.const_uploaded = True
        self.last_h2d_bytes = (hi - lo) * 4

    # -- device side -----------------------------------------------------------------
    def _forward(self) -> None:
        eng = self.engine
        self.logits = eng.model.forward(self.ctx)
        self.next_tokens = ops.sample(self.logits, self.v_temperature, self.v_top_k, self.v_top_p, self.v_stream,
                                      self.v_counter, eng.sampler.seed)
        self.v_tokens.copy_(self.next_tokens)          # the chosen token is the next step's input

    def run(self, req_ids: Sequence, tokens: Optional[Sequence[int]], temperature, top_k, top_p, stream_ids,
            counters) -> torch.Tensor:
        """One decode step of ``req_ids`` (pages already reserved).  ``tokens`` None:
        the ids chosen by the previous run are still on the device and are used.
        Fewer requests than the graph's batch size are padded (see ``_fill``).
        Returns the chosen tokens, int32 [len(req_ids)] on the device (valid until the next run)."""
        assert len(req_ids) == self.B or (len(req_ids) < self.B and self.engine.cache.scratch_pages() is not None)
        self._fill(req_ids, tokens, temperature, top_k, top_p, stream_ids, counters)
        self._upload(with_tokens=tokens is not None)
        self.uses += 1
        if self.graph is None:
            before = ops.launch_count()
            self._forward()                                                      # this step runs eagerly
            self.kernels_per_replay = ops.launch_count() - before
            result = self.next_tokens
            self._capture()
            return result[:len(req_ids)]
        self.graph.replay()
        ops.count_launches(self.kernels_per_replay)
        return self.next_tokens[:len(req_ids)]

    def _capture(self) -> None:
        """Capture the step for later replays.  Nothing runs during capture; the
        cache and the token buffer are not touched."""
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        # No cyclic garbage collection while the stream captures: what it frees may be another engine's captured
        # graphs, and destroying a graph is not permitted during a capture (it invalidates this one).
        gc_was_on = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            with torch.cuda.graph(g):
                self._forward()
        finally:
            if gc_was_on:
                gc.enable()
        self.graph = g
