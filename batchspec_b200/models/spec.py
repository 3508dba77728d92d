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
    """One layer: the kind of its block, one part per slot that the block kind
    declares (``Block.SLOTS``), and the checkpoint name of each local tensor name,
    keyed ``"<slot>.<local>"``."""
    parts: Dict[str, PartSpec]
    names: Dict[str, str]
    block: str = "prenorm"


def prenorm_layer(norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, ffn: PartSpec, names: Dict[str, str]) -> LayerSpec:
    """The pre-norm residual layer: norm -> mixer -> add, norm -> feed-forward -> add."""
    return LayerSpec({"norm1": norm1, "mixer": mixer, "norm2": norm2, "ffn": ffn}, names, "prenorm")


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
    must_equal: Dict[str, str] = field(default_factory=dict)   # tensor that may be absent -> the tensor it must copy
    embed_scale: float = 1.0
    # optional parts that run once per step: after the embedding (registry INPUT_PARTS) and on the head's
    # output (LOGITS_PARTS), each with the checkpoint names of its tensors
    input_part: Optional[PartSpec] = None
    input_names: Dict[str, str] = field(default_factory=dict)
    logits_part: Optional[PartSpec] = None
    logits_names: Dict[str, str] = field(default_factory=dict)
