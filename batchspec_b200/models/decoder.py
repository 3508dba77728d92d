"""Generic executor of a ``ModelSpec``: embedding (then the optional input part),
the listed runs of layers, final norm, head over the wanted rows only (then the
optional logits part).

The reference computes logits for every token of the step and then selects the
last row of each request (batchspec/models/standard_model.py:90-102,
backends/standard_engine.py:127); here only the rows asked for reach the head."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from ..parts.base import (BLOCKS, INPUT_PARTS, LOGITS_PARTS, NORMS, CacheSpec, ParamSpec, Runtime, StateSpec,
                          build_part)
from .spec import ModelSpec


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache.  ``kv``: [pages, tensors per token,
    page_size * entry elements] of its group's pool (None if the mixer asked for no pages);
    ``group``: index of the block tables in the step context; ``state``:
    [max_requests, *state_shape] or None; ``owner``: False for a run that reads
    another run's cache."""
    kv: Optional[torch.Tensor]
    group: int
    state: Optional[torch.Tensor]
    owner: bool


@dataclass
class CacheNeed:
    """Per run of the order: what its mixer asks for and whose cache it uses."""
    cache: Optional[CacheSpec]
    state: Optional[StateSpec]
    cache_from: Optional[int]


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.runtime = spec, runtime
        self.blocks = []
        for i, layer in enumerate(spec.layers):
            if layer.block not in BLOCKS:
                raise KeyError(f"block kind {layer.block!r} is not registered (known: {sorted(BLOCKS)})")
            kind = BLOCKS[layer.block]
            if set(layer.parts) != set(kind.SLOTS):
                raise ValueError(f"layer {i}: block {layer.block!r} has slots {list(kind.SLOTS)}, "
                                 f"the description gives {list(layer.parts)}")
            self.blocks.append(kind(**{slot: build_part(registry, layer.parts[slot], runtime)
                                       for slot, registry in kind.SLOTS.items()}))
        self.final_norm = build_part(NORMS, spec.final_norm, runtime)
        self.input_part = build_part(INPUT_PARTS, spec.input_part, runtime) if spec.input_part else None
        self.logits_part = build_part(LOGITS_PARTS, spec.logits_part, runtime) if spec.logits_part else None
        for e, run in enumerate(spec.order):
            if not 0 <= run.layer < len(spec.layers):
                raise ValueError(f"order[{e}] names layer {run.layer}, the model has {len(spec.layers)}")
            if run.cache_from is not None:
                if not 0 <= run.cache_from < e or spec.order[run.cache_from].cache_from is not None:
                    raise ValueError(f"order[{e}].cache_from must name an earlier run that owns its cache")
        self.embed: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None
        self.caches: List[Optional[LayerCache]] = [None] * len(spec.order)

    @property
    def graph_safe(self) -> bool:
        parts = [self.final_norm, self.input_part, self.logits_part]
        for b in self.blocks:
            for part in b.parts.values():
                parts += [part, getattr(part, "position", None)]
        return all(getattr(p, "graph_safe", False) for p in parts if p is not None)

    # -- tensors ---------------------------------------------------------------
    def _named_parts(self):
        """(what it is, part, local name -> checkpoint name) of every part that holds tensors, in a fixed order."""
        s = self.spec
        if self.input_part is not None:
            yield "input part", self.input_part, s.input_names
        for i, layer in enumerate(s.layers):
            for slot, part in self.blocks[i].parts.items():
                yield f"layer {i}", part, {local: layer.names.get(f"{slot}.{local}") for local in part.param_specs()}, f"{slot}."
        yield "final norm", self.final_norm, s.final_norm_names
        if self.logits_part is not None:
            yield "logits part", self.logits_part, s.logits_names

    def param_specs(self) -> Dict[str, ParamSpec]:
        """checkpoint name -> ParamSpec, in a fixed order."""
        s = self.spec
        out = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for where, part, names, *prefix in self._named_parts():
            for local, ps in part.param_specs().items():
                if names.get(local) is None:
                    raise KeyError(f"{where}: no checkpoint name given for '{(prefix[0] if prefix else '') + local}'")
                out[names[local]] = ps
        if s.lm_head_name is not None:
            out[s.lm_head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = tensors[s.embed_name]
        for where, part, names, *prefix in self._named_parts():
            part.bind({local: tensors[names[local]] for local in part.param_specs()})
        self.head = self.embed if s.lm_head_name is None else tensors[s.lm_head_name]

    # -- cache -----------------------------------------------------------------
    def cache_needs(self) -> List[CacheNeed]:
        out = []
        for run in self.spec.order:
            block = self.blocks[run.layer]
            mixer = getattr(block, block.MIXER_SLOT)
            out.append(CacheNeed(mixer.cache_spec(), mixer.state_spec(), run.cache_from))
        return out

    def attach_caches(self, caches: List[Optional[LayerCache]]) -> None:
        assert len(caches) == len(self.spec.order)
        self.caches = list(caches)

    # -- one step --------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """ctx: the step context (token ids, positions, tables, wanted rows).
        Returns float32 logits [len(ctx.logit_rows), vocab]."""
        s = self.spec
        n = ctx.n_tokens
        resid = torch.empty((n, s.hidden_size), dtype=torch.float32, device=self.runtime.device)
        with bucket("embed"):
            ops.embed(ctx.token_ids, self.embed, resid, s.embed_scale)
        if self.input_part is not None:
            self.input_part.forward(resid, ctx)
        pending = None
        for e, run in enumerate(s.order):
            resid, pending = self.blocks[run.layer].forward(resid, pending, ctx, self.caches[e])
        n_out = ctx.n_logit_rows
        if n_out == 0:
            return torch.empty((0, s.vocab_size), dtype=torch.float32, device=self.runtime.device)
        picked = torch.empty((n_out, s.hidden_size), dtype=torch.float32, device=self.runtime.device)
        ops.gather_rows_add(resid, pending, ctx.logit_rows, picked)
        z = self.final_norm.forward(picked, None)
        with bucket("lm_head"):
            logits = ops.linear(z, self.head, out_dtype=torch.float32)
        if self.logits_part is not None:
            self.logits_part.forward(logits, ctx)
        return logits
