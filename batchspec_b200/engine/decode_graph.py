"""Decode steps as CUDA graphs.

A step in which every entry is one token of a live request has the same kernels
and launch sizes whenever the number of entries is the same; only the metadata
(positions, block tables, state slots, sampling counters) and the token ids
differ.  ``DecodeGraph`` keeps that metadata in one device buffer with a fixed
layout, captures model forward + sampling once per batch size, and replays it
with a fresh upload per step.  The kernels read everything that changes from the
buffer, never from launch arguments.  This replaces the reference's
``torch.compile`` of the step (batchspec/backends/standard_engine.py:103-106).

Layout of the int32 metadata buffer for B entries and at most P pages per request
(``dyn`` is uploaded every step, the tables only when a page was added):

    dyn:    token_ids[B] positions[B] kv_len[B] state_slots[B] top_k[B]
            temperature[B] (f32) top_p[B] (f32) stream_id[B] (i64) counter[B] (i64)
    const:  tok_entry[B] qo_indptr[B+1] logit_rows[B] kv_indptr[B+1] (per group)
    tables: kv_indices[B * P] per group
"""
from __future__ import annotations

import gc

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .step import GroupTables, StepContext


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class DecodeGraph:
    def __init__(self, engine, batch: int, max_pages: int, max_kv_len: int):
        self.engine, self.B, self.P = engine, int(batch), int(max_pages)
        self.max_kv_len = int(max_kv_len)
        cache = engine.cache
        B, P, ng = self.B, self.P, len(cache.groups)
        off, o = {}, 0
        for name in ("token_ids", "positions", "kv_len", "state_slots", "top_k", "temperature", "top_p"):
            off[name] = o
            o += _align(B)
        o = _align(o, 2)
        for name in ("stream_id", "counter"):
            off[name] = o
            o += _align(2 * B)
        self.dyn_len = o
        for name in ("tok_entry", "logit_rows"):
            off[name] = o
            o += _align(B)
        off["qo_indptr"] = o
        o += _align(B + 1)
        for g in range(ng):
            off[f"kv_indptr{g}"] = o
            o += _align(B + 1)
        self.table_begin = o
        for g in range(ng):
            off[f"kv_indices{g}"] = o
            o += _align(B * P)
        self.total = o
        self.off = off
        self.meta = np.zeros(self.total, dtype=np.int32)                 # the authoritative host copy
        self.meta[off["tok_entry"]:off["tok_entry"] + B] = np.arange(B)
        self.meta[off["logit_rows"]:off["logit_rows"] + B] = np.arange(B)
        self.meta[off["qo_indptr"]:off["qo_indptr"] + B + 1] = np.arange(B + 1)
        for g in range(ng):
            self.meta[off[f"kv_indptr{g}"]:off[f"kv_indptr{g}"] + B + 1] = np.arange(B + 1) * P
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
        self.v_tokens = view("token_ids", B)
        self.v_temperature, self.v_top_p = f32("temperature"), f32("top_p")
        self.v_top_k = view("top_k", B)
        self.v_stream, self.v_counter = i64("stream_id"), i64("counter")
        tables = [GroupTables(cache.page_size, view(f"kv_indptr{g}", B + 1), view(f"kv_indices{g}", B * P), None, None)
                  for g in range(ng)]
        self.ctx = StepContext(
            n_tokens=B, n_entries=B, token_ids=self.v_tokens, positions=view("positions", B),
            tok_entry=view("tok_entry", B), qo_indptr=view("qo_indptr", B + 1), kv_len=view("kv_len", B),
            state_slots=view("state_slots", B), logit_rows=view("logit_rows", B), n_logit_rows=B, tables=tables,
            max_q_len=1, max_kv_len=self.max_kv_len, h_qo_indptr=None, h_kv_len=None, h_state_slots=None,
            h_positions=None, extras={"min_q_len": 1, "captured": True})

    # -- host side -------------------------------------------------------------------
    _PAD = object()        # marks a table row that currently points at the scratch page

    def _fill(self, req_ids: Sequence, tokens: Optional[Sequence[int]], temperature, top_k, top_p, stream_ids,
              counters) -> None:
        cache, off, B, P, m = self.engine.cache, self.off, self.B, self.P, self.meta
        n = len(req_ids)
        reqs = [cache.requests[r] for r in req_ids]
        # rows n .. B-1 are padding: one token at position 0 of the scratch page, greedy, result ignored
        lengths = np.zeros(B, dtype=np.int32)
        lengths[:n] = [rc.length for rc in reqs]

        def put(name, values, view=None, width=1):
            dst = m[off[name]:off[name] + width * B]
            if view is not None:
                dst = dst.view(view)
            dst[:n] = values
            dst[n:] = 0

        if tokens is not None:
            put("token_ids", tokens)
        m[off["positions"]:off["positions"] + B] = lengths
        m[off["kv_len"]:off["kv_len"] + B] = lengths + 1
        put("state_slots", [rc.slot for rc in reqs])
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
                        m[off[f"kv_indices{g}"] + i * P] = page
                        self.row_pages[i][g] = 0
                    self.row_req[i] = self._PAD
                    self.tables_dirty = True
        for i, (rid, rc) in enumerate(zip(req_ids, reqs)):
            # the row's table on the device is this request's only if it is the same admission: a request that was
            # preempted and admitted again has the same id but other pages (perhaps as many as before)
            fresh = self.row_req[i] != (rid, rc.serial)
            for g, table in enumerate(rc.tables):
                have = 0 if fresh else self.row_pages[i][g]
                if len(table) > P:
                    raise RuntimeError(f"request {rid!r} holds {len(table)} pages, the captured step allows {P}")
                if fresh or len(table) != have:
                    base = off[f"kv_indices{g}"] + i * P
                    lo = 0 if fresh or len(table) < have else have
                    m[base + lo:base + len(table)] = table[lo:]
                    self.row_pages[i][g] = len(table)
                    self.tables_dirty = True
                elif cache.groups[g].spec.policy == "window":
                    base = off[f"kv_indices{g}"] + i * P        # released pages turn into -1 in place
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
        lo = 0 if with_tokens else _align(B)
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
