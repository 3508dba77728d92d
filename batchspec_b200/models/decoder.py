"""Generic executor of a ``ModelSpec``: embedding, the listed runs of layers,
final norm, head over the wanted rows only.

The reference computes logits for every token of the step and then selects the
last row of each request (batchspec/models/standard_model.py:90-102,
backends/standard_engine.py:127); here only the rows asked for reach the head."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheSpec, ParamSpec, Runtime, StateSpec,
                          build_part)
from .spec import ModelSpec


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache.  ``kv``: [pages, 2, page_size,
    *entry_shape] of its group's pool (None if the mixer asked for no pages);
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
        for layer in spec.layers:
            if layer.block not in BLOCKS:
                raise KeyError(f"block kind {layer.block!r} is not registered (known: {sorted(BLOCKS)})")
            self.blocks.append(BLOCKS[layer.block](
                build_part(NORMS, layer.norm1, runtime), build_part(MIXERS, layer.mixer, runtime),
                build_part(NORMS, layer.norm2, runtime), build_part(FEED_FORWARDS, layer.ffn, runtime)))
        self.final_norm = build_part(NORMS, spec.final_norm, runtime)
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
        parts = [self.final_norm]
        for b in self.blocks:
            parts += [b.norm1, b.mixer, b.norm2, b.ffn, getattr(b.mixer, "position", None)]
        return all(getattr(p, "graph_safe", False) for p in parts if p is not None)

    # -- tensors ---------------------------------------------------------------
    def _slots(self, i):
        b = self.blocks[i]
        return {"norm1": b.norm1, "mixer": b.mixer, "norm2": b.norm2, "ffn": b.ffn}

    def param_specs(self) -> Dict[str, ParamSpec]:
        """checkpoint name -> ParamSpec, in a fixed order."""
        s = self.spec
        out = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for i, layer in enumerate(s.layers):
            for slot, part in self._slots(i).items():
                for local, ps in part.param_specs().items():
                    key = f"{slot}.{local}"
                    if key not in layer.names:
                        raise KeyError(f"layer {i}: no checkpoint name given for '{key}'")
                    out[layer.names[key]] = ps
        for local, ps in self.final_norm.param_specs().items():
            out[s.final_norm_names[local]] = ps
        if s.lm_head_name is not None:
            out[s.lm_head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = tensors[s.embed_name]
        for i, layer in enumerate(s.layers):
            for slot, part in self._slots(i).items():
                part.bind({local: tensors[layer.names[f"{slot}.{local}"]] for local in part.param_specs()})
        self.final_norm.bind({local: tensors[s.final_norm_names[local]] for local in self.final_norm.param_specs()})
        self.head = self.embed if s.lm_head_name is None else tensors[s.lm_head_name]

    # -- cache -----------------------------------------------------------------
    def cache_needs(self) -> List[CacheNeed]:
        out = []
        for run in self.spec.order:
            mixer = self.blocks[run.layer].mixer
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
            return ops.linear(z, self.head, out_dtype=torch.float32)
