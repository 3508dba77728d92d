"""Interfaces of the parts a decoder is assembled from, and their registries.

A *part* is a parametrised object that knows its own sizes and constants and
nothing about the model it sits in: it names its tensors by short local names
(``q``, ``gate`` ...), the architecture supplies the map from local names to
checkpoint names.  The reference fixes the parts by subclass hooks
(batchspec/models/base_model.py:138-173, ``_get_attention_class`` /
``_get_block_class``); here they are chosen per layer by the model description, so
one model may mix different mixers and feed-forwards.

Registries: ``MIXERS``, ``FEED_FORWARDS``, ``NORMS``, ``POSITION_ENCODINGS``,
``BLOCKS``, ``INPUT_PARTS``, ``LOGITS_PARTS``.  ``register_part(registry, kind)``
is a class decorator; ``build_part(registry, spec, runtime)`` instantiates
``spec.kind`` with ``spec.params``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class PartSpec:
    """Which part (``kind``) and with which sizes/constants (``params``)."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    role: ``matrix`` (a GEMM operand or lookup table: held in the run dtype),
          ``vector`` (a per-channel scale: held in the run dtype unless the file
          stores it in 32-bit, which is kept), ``int`` (an integer table: int32).
    init: ``normal`` -> N(0, std);  ``ones_normal`` -> 1 + N(0, std).
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer asks of the paged cache, per token and per layer.

    policy ``full``: every token's entry is kept while the request lives.
    policy ``window``: only the last ``window`` tokens are ever read; pages that
    lie wholly before the window are given back.
    ``entry_shape`` is the per-token shape of ONE stored tensor, e.g.
    (n_kv_heads, head_dim); ``tensors`` says how many of them a token has: 2 for
    keys and values, 1 for a mixer that stores a single (compressed) entry.
    ``page_size``: tokens per page of this mixer's group, or None for the
    engine's default; groups with different page sizes have block tables of
    different lengths for the same request."""
    policy: str
    entry_shape: Tuple[int, ...]
    window: Optional[int] = None
    tensors: int = 2
    page_size: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer (a recurrent state, a conv tail):
    one tensor of ``shape``/``dtype`` per live request, zeroed when a request is
    admitted, addressed by the request's state slot."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What every part gets at construction: run dtype and device."""
    dtype: torch.dtype
    device: torch.device


class Part:
    """Common protocol.  ``param_specs`` -> local name -> ParamSpec;
    ``bind`` receives the loaded tensors (on the device) under those names.
    ``graph_safe``: True if ``forward`` only enqueues device work whose launch
    sizes depend on the number of tokens and entries alone and reads everything
    else from the step context's device tensors; such parts may be captured in a
    CUDA graph.  A part that reads host fields of the context must leave it False."""
    graph_safe = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        pass


class Norm(Part):
    """``forward(resid, delta, out=None)``: ``resid`` is the float32 residual
    stream [n, d]; if ``delta`` is given it is first added into ``resid`` in
    place (the residual sum, in 32-bit); returns the normalised rows in the run
    dtype."""

    def forward(self, resid: torch.Tensor, delta: Optional[torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """``apply(q, k, ctx)`` rotates/offsets q [n, Hq, hd] and k [n, Hkv, hd] (views,
    in place) for the tokens' absolute positions ``ctx.positions``.  A part that
    can be folded into the attention mixer's fused rotate-and-append kernel also
    offers ``rope_table()`` -> (``ops.rope_frequency_table`` of rotary_dim/2 frequencies, rotary_dim,
    interleaved)."""

    def apply(self, q: torch.Tensor, k: torch.Tensor, ctx) -> None:
        raise NotImplementedError

    def rope_table(self):
        return None


class Mixer(Part):
    """Token mixer.  ``forward(x, ctx, cache)``: x [n, d] run dtype -> [n, d].
    ``cache`` is the LayerCache the model description assigned to this run of the
    layer (None if the mixer declared no needs): ``cache.kv`` the layer's page
    tensor and ``cache.group`` the index of its block tables in ``ctx``,
    ``cache.state`` its per-request state tensor [max_requests, *shape],
    ``cache.owner`` False when the layer only reads another layer's cache."""

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, ctx)``: x [n, d] run dtype -> [n, d]."""

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class InputPart(Part):
    """Runs once per step right after the embedding: ``forward(resid, ctx)`` changes
    the float32 residual rows [n, d] in place (a learned absolute position row
    added to each token, a multiplier ...)."""

    def forward(self, resid: torch.Tensor, ctx) -> None:
        raise NotImplementedError


class LogitsPart(Part):
    """Runs once per step on the head's output: ``forward(logits, ctx)`` changes the
    float32 logits [wanted rows, vocab] in place (a scale, a soft cap ...)."""

    def forward(self, logits: torch.Tensor, ctx) -> None:
        raise NotImplementedError


MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}
INPUT_PARTS: Dict[str, type] = {}
LOGITS_PARTS: Dict[str, type] = {}


class Block:
    """Arrangement of a layer's parts around the residual stream.  A block kind
    declares its slots as data: ``SLOTS`` maps slot name -> the registry its part
    comes from, in the order the parts' tensors are listed; the model description
    gives one ``PartSpec`` per slot.  ``MIXER_SLOT`` names the slot whose part
    (a ``Mixer``) owns the layer's cache and per-request state.  The built parts
    arrive as keyword arguments and are kept as attributes of the same names and in
    ``self.parts``.

    ``forward(resid, pending, ctx, cache)`` takes the float32 residual and a
    not-yet-added branch output (or None) and returns the same pair, so the add
    can be fused into the next norm."""
    SLOTS: Dict[str, Dict[str, type]] = {}
    MIXER_SLOT = "mixer"

    def __init__(self, **parts):
        missing, extra = set(self.SLOTS) - set(parts), set(parts) - set(self.SLOTS)
        if missing or extra:
            raise ValueError(f"block {type(self).__name__} has slots {list(self.SLOTS)}; missing {sorted(missing)}, "
                             f"unexpected {sorted(extra)}")
        self.parts = {slot: parts[slot] for slot in self.SLOTS}
        for slot, part in self.parts.items():
            setattr(self, slot, part)

    def forward(self, resid, pending, ctx, cache):
        raise NotImplementedError


def register_part(registry: Dict[str, type], kind: str):
    def deco(cls):
        registry[kind] = cls
        cls.kind = kind
        return cls
    return deco


def build_part(registry: Dict[str, type], spec: PartSpec, runtime: Runtime):
    if spec.kind not in registry:
        raise KeyError(f"part kind {spec.kind!r} is not registered (known: {sorted(registry)})")
    return registry[spec.kind](runtime=runtime, **spec.params)
