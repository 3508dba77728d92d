"""The step function: one batch of (request, its next tokens) through the model.

The reference's step is ``StandardEngine.forward(batch)`` over a ``BatchPack``
(batchspec/backends/standard_engine.py:109-128, backends/continuous/batch_builder.py:30-81):
exactly one entry per batch slot, dummy entries for empty slots, logits for every
token, then the last row of each slot.  Here a step holds any number of entries,
each ``n >= 1`` new tokens of a live request (a portion of a prompt or a decoded
token, cut anywhere), runs only those tokens against the cache that earlier steps
left, and returns float32 logits at the places asked for.

Order inside a step: reserve pages for every entry (all or nothing) -> pack the
metadata into one pinned buffer and copy it once -> model forward -> commit the
new lengths.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager


@dataclass
class StepEntry:
    """``tokens``: the request's next tokens; ``want``: indices into ``tokens``
    whose logits are returned (may be empty)."""
    req_id: object
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GroupTables:
    """Block tables of one cache group for the entries of the step, as CSR."""
    page_size: int
    kv_indptr: torch.Tensor            # int32 [n_entries + 1]
    kv_indices: torch.Tensor           # int32 [sum of table lengths], -1 for released pages
    h_kv_indptr: np.ndarray
    h_kv_indices: np.ndarray


# The int32 fields of a step's metadata, in packing order, each with the count that gives its length.  Both
# ways of running a step (the packed buffer below, the fixed layout of a captured decode step) take this list
# and ``step_fields``: a new field is added here, there and to ``StepContext``, nowhere else.
CONTEXT_FIELDS = (("token_ids", "tokens"), ("positions", "tokens"), ("tok_entry", "tokens"), ("qo_indptr", "entries+1"),
                  ("kv_len", "entries"), ("state_slots", "entries"), ("logit_rows", "rows"))


def field_length(kind: str, n_tokens: int, n_entries: int, n_rows: int) -> int:
    return {"tokens": n_tokens, "entries": n_entries, "entries+1": n_entries + 1, "rows": n_rows}[kind]


def step_fields(cache: CacheManager, req_ids: Sequence, lens: Sequence[int], wants: Sequence[Sequence[int]],
                tokens: Optional[Sequence[Sequence[int]]] = None, with_tables: bool = True):
    """The values of ``CONTEXT_FIELDS`` for a step of these entries, and per cache group the entries' block
    tables as CSR (indptr, indices).  ``req_ids[i]`` None is a padding entry: a request of length 0 in the
    cache's scratch state slot whose table is the scratch page.  ``tokens`` None: the ids are already on the
    device and ``token_ids`` comes back empty.  ``with_tables`` False: no tables (the caller keeps its own copy
    of them up to date)."""
    n = len(req_ids)
    reqs = [cache.requests[r] if r is not None else None for r in req_ids]
    lens = np.asarray(lens, dtype=np.int64).reshape(n)
    before = np.fromiter((rc.length if rc is not None else 0 for rc in reqs), dtype=np.int64, count=n)
    qo = np.zeros(n + 1, dtype=np.int32)
    np.cumsum(lens, out=qo[1:])
    nnz = int(qo[-1])
    if tokens is not None:
        ids = np.concatenate([np.asarray(t, dtype=np.int64).reshape(-1) for t in tokens]) if n else np.zeros(0, np.int64)
    else:
        ids = np.zeros(0, dtype=np.int64)
    pad_slot = cache.scratch_slot()
    rows: List[int] = []
    for i, want in enumerate(wants):
        for w in want:
            if not 0 <= w < lens[i]:
                raise ValueError(f"request {req_ids[i]!r}: wanted place {w} is outside its {lens[i]} tokens")
            rows.append(int(qo[i]) + int(w))
    fields = {
        "token_ids": ids.astype(np.int32),
        "positions": (np.arange(nnz, dtype=np.int64) - np.repeat(qo[:-1].astype(np.int64), lens)
                      + np.repeat(before, lens)).astype(np.int32),
        "tok_entry": np.repeat(np.arange(n, dtype=np.int32), lens),
        "qo_indptr": qo,
        "kv_len": (before + lens).astype(np.int32),
        "state_slots": np.fromiter((rc.slot if rc is not None else (pad_slot or 0) for rc in reqs), dtype=np.int32, count=n),
        "logit_rows": np.asarray(rows, dtype=np.int32),
    }
    scratch = cache.scratch_pages()
    tables = []
    for gi in range(len(cache.groups) if with_tables else 0):
        tabs = [rc.tables[gi] if rc is not None else [scratch[gi]] for rc in reqs]
        indptr = np.zeros(n + 1, dtype=np.int32)
        np.cumsum([len(t) for t in tabs], out=indptr[1:])
        tables.append((indptr, np.fromiter((p for t in tabs for p in t), dtype=np.int32, count=int(indptr[-1]))))
    return fields, tables


@dataclass
class StepContext:
    """Everything the parts may read about the step.  Device tensors are int32
    views into one buffer; ``host`` holds the same values on the host under the same names (None for a captured
    step, whose values change from replay to replay), also readable as ``h_<name>``."""
    n_tokens: int
    n_entries: int
    token_ids: torch.Tensor            # [n_tokens]
    positions: torch.Tensor            # [n_tokens] absolute position of each token in its request
    tok_entry: torch.Tensor            # [n_tokens] index of the token's entry
    qo_indptr: torch.Tensor            # [n_entries + 1]
    kv_len: torch.Tensor               # [n_entries] request length after this step
    state_slots: torch.Tensor          # [n_entries] state slot of each entry's request
    logit_rows: torch.Tensor           # [n_logit_rows] flat token indices whose logits are wanted
    n_logit_rows: int
    tables: List[GroupTables]
    max_q_len: int
    max_kv_len: int
    host: Optional[dict] = None
    extras: dict = field(default_factory=dict)

    def __getattr__(self, name):
        if name.startswith("h_"):
            host = self.__dict__.get("host")
            return None if host is None else host[name[2:]]
        raise AttributeError(name)


class _Staging:
    """Pinned host buffers (a small ring) and one device buffer for the packed
    metadata.  A host buffer is rewritten only after the copy that last read it
    has finished."""

    def __init__(self, device, capacity: int = 1 << 16, ring: int = 3):
        self.device = device
        self.ring = ring
        self.capacity = 0
        self._grow(capacity)

    def _grow(self, capacity: int) -> None:
        if self.capacity:
            torch.cuda.current_stream().synchronize()
        self.capacity = capacity
        pin = self.device.type == "cuda"
        self.host = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(self.ring)]
        self.dev = [torch.empty(capacity, dtype=torch.int32, device=self.device) for _ in range(self.ring)]
        self.events = [None] * self.ring
        self.turn = 0

    def upload(self, packed: np.ndarray) -> torch.Tensor:
        n = packed.shape[0]
        if n > self.capacity:
            self._grow(max(n, 2 * self.capacity))
        i = self.turn
        self.turn = (self.turn + 1) % self.ring
        if self.events[i] is not None:
            self.events[i].synchronize()
        self.host[i].numpy()[:n] = packed
        self.dev[i][:n].copy_(self.host[i][:n], non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self.events[i] = ev
        return self.dev[i]


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepRunner:
    def __init__(self, model, cache: CacheManager, vocab_size: int, device):
        self.model, self.cache, self.vocab_size = model, cache, int(vocab_size)
        self.device = torch.device(device)
        self.staging = _Staging(self.device)
        self.last_h2d_bytes = 0

    def build_context(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> StepContext:
        """Pack the metadata of a step whose pages are already reserved.  With
        ``device_tokens`` (int32 [n_tokens], already on the device) the entries'
        token values are not looked at, only their counts."""
        cache = self.cache
        n = len(entries)
        lens = [len(e.tokens) for e in entries]
        fields, group_tables = step_fields(cache, [e.req_id for e in entries], lens, [e.want for e in entries],
                                           None if device_tokens is not None else [e.tokens for e in entries])
        ids = fields["token_ids"]
        if ids.size and (ids.min() < 0 or ids.max() >= self.vocab_size):
            raise ValueError(f"token id outside [0, {self.vocab_size}) in the step")
        names = [name for name, _ in CONTEXT_FIELDS]
        parts = [fields[name] for name in names]
        for indptr, indices in group_tables:
            parts += [indptr, indices]
        offsets, total = [], 0
        for p in parts:
            offsets.append(total)
            total += _align4(max(p.shape[0], 1))
        packed = np.zeros(total, dtype=np.int32)
        for o, p in zip(offsets, parts):
            packed[o:o + p.shape[0]] = p
        dev = self.staging.upload(packed)
        self.last_h2d_bytes = total * 4
        view = lambda k: dev[offsets[k]:offsets[k] + parts[k].shape[0]]
        views = {name: view(k) for k, name in enumerate(names)}
        if device_tokens is not None:
            views["token_ids"] = device_tokens
        tables = []
        for gi, g in enumerate(cache.groups):
            k = len(names) + 2 * gi
            tables.append(GroupTables(g.page_size, view(k), view(k + 1), group_tables[gi][0], group_tables[gi][1]))
        return StepContext(
            n_tokens=int(fields["qo_indptr"][-1]), n_entries=n, n_logit_rows=int(fields["logit_rows"].shape[0]),
            tables=tables, max_q_len=max(lens), max_kv_len=int(fields["kv_len"].max()), host=fields,
            extras={"min_q_len": min(lens)}, **views)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run the entries as one batch; float32 logits [sum of len(want), vocab] in
        the order of the entries and of their ``want``."""
        cache = self.cache
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if len(e.tokens) < 1:
                raise ValueError(f"request {e.req_id!r}: an entry needs at least one token")
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            if not cache.is_live(e.req_id):
                raise KeyError(f"request {e.req_id!r} is not live (admit it first)")
        need = [0] * len(cache.groups)                    # per group; pages held ahead count as held
        for e in entries:
            need = [a + b for a, b in zip(need, cache.pages_missing(e.req_id, len(e.tokens)))]
        if any(n > g.pool.num_free for n, g in zip(need, cache.groups)):
            from ..cache.manager import OutOfPages
            raise OutOfPages("the step needs more pages than are free; nothing was run")
        for e in entries:
            cache.reserve(e.req_id, len(e.tokens))
        ctx = self.build_context(entries, device_tokens)
        logits = self.model.forward(ctx)
        for e in entries:
            cache.commit(e.req_id, len(e.tokens))
        return logits
