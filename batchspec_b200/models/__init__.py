"""Registry from an architecture's name to its model builder.

The reference maps a *type* (standard / eagle / mtp) to a class
(batchspec/models/__init__.py:101-142); here the key is ``architectures[0]`` of
config.json and the value a function from that architecture's configuration to a
``ModelSpec``."""
from __future__ import annotations

from typing import Callable, Dict

from ..parts.base import Runtime
from .decoder import CacheNeed, DecoderModel, LayerCache
from .llama import build_llama
from .spec import LayerSpec, ModelSpec, RunEntry, prenorm_layer

MODEL_REGISTRY: Dict[str, Callable] = {}


def register_model(architecture: str, builder: Callable) -> None:
    MODEL_REGISTRY[architecture] = builder


def get_model(config, runtime: Runtime) -> DecoderModel:
    arch = config.architecture
    if arch not in MODEL_REGISTRY:
        raise KeyError(f"architecture {arch!r} has no registered model (known: {sorted(MODEL_REGISTRY)})")
    return DecoderModel(MODEL_REGISTRY[arch](config), runtime)


register_model("LlamaForCausalLM", build_llama)

__all__ = ["MODEL_REGISTRY", "register_model", "get_model", "DecoderModel", "LayerCache", "CacheNeed",
           "ModelSpec", "LayerSpec", "RunEntry", "prenorm_layer", "build_llama"]
