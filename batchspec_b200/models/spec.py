"""The description of a decoder as data: which parts each layer is made of, the
order in which layers run, which cache each run uses, and the checkpoint names of
every tensor.  An architecture's builder turns its configuration into one of
these; the generic ``DecoderModel`` executes it."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..parts.base import PartSpec


@dataclass
class LayerSpec:
    """One layer: its parts and the checkpoint name of each local tensor name,
    keyed ``"<slot>.<local>"`` with slot in norm1 / mixer / norm2 / ffn."""
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    ffn: PartSpec
    names: Dict[str, str]
    block: str = "prenorm"


@dataclass
class RunEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers`` (the same layer
    may be run more than once: shared weights, separate caches).  ``cache_from``
    is None when the run owns a cache of its own, or the index of an EARLIER entry
    of the order whose cache this run reads without writing."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    vocab_size: int
    hidden_size: int
    layers: List[LayerSpec]
    order: List[RunEntry]
    final_norm: PartSpec
    embed_name: str
    final_norm_names: Dict[str, str]
    lm_head_name: Optional[str]          # None: the head is the embedding table (tied)
    ignore_suffixes: Tuple[str, ...] = ()
    ignore_names: Tuple[str, ...] = ()
    embed_scale: float = 1.0
