"""The engine: model + cache + step function + generation loop.

Method names follow the reference's ``StandardEngine``
(batchspec/backends/standard_engine.py:17-172, backends/base/engine.py:13-147):
``load_model`` -> ``setup_caches`` -> ``setup_sampling_params`` -> ``generate``.
What differs: the model comes from a folder with ``config.json`` and safetensors
(or random weights from a seed), the cache is a shared page pool instead of a
static range per slot, ``step`` is public and returns logits, and sampling is a
separate call.
"""
from __future__ import annotations

from pathlib import Path
from typing import List, Optional, Sequence

import torch

from ..cache.manager import CacheManager
from ..config import get_config, load_config
from ..models import get_model
from ..parts.base import Runtime
from ..weights import load_weights, random_weights
from .step import StepEntry, StepRunner

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {dtype}")
        return dtype
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    return _DTYPES[dtype]


class Engine:
    def __init__(self, dtype="bfloat16", device="cuda:0", tokenizer=None):
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("batchspec_b200 runs on a CUDA device (sm_100a) only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is available; batchspec_b200 has no CPU path")
        self.tokenizer = tokenizer
        self.config = None
        self.model = None
        self.cache: Optional[CacheManager] = None
        self.runner: Optional[StepRunner] = None
        self.page_size = None

    # -- model -------------------------------------------------------------------
    def load_model(self, model_dir=None, config=None, config_name: Optional[str] = None,
                   random_seed: Optional[int] = None, draw_on_device: bool = False,
                   stored_dtype: Optional[torch.dtype] = None) -> None:
        """Either ``model_dir`` (config.json + safetensors), or a configuration
        (``config`` object or ``config_name`` of the by-name table) with
        ``random_seed`` for random weights."""
        from ..kernels import ops
        ops.load_library()
        torch.cuda.set_device(self.device)
        runtime = Runtime(self.dtype, self.device)
        if model_dir is not None:
            self.config = load_config(model_dir)
            self.model = get_model(self.config, runtime)
            s = self.model.spec
            tensors = load_weights(model_dir, self.model.param_specs(), self.dtype, self.device,
                                   ignore_suffixes=s.ignore_suffixes, ignore_names=s.ignore_names)
        else:
            if config is None:
                if config_name is None:
                    raise ValueError("give model_dir, config or config_name")
                config = get_config(config_name)
            if random_seed is None:
                raise ValueError("a configuration without a folder needs random_seed")
            self.config = config
            self.model = get_model(config, runtime)
            tensors = random_weights(self.model.param_specs(), random_seed, self.dtype, self.device,
                                     draw_on_device=draw_on_device, stored_dtype=stored_dtype)
        self.model.bind(tensors)

    # -- cache -------------------------------------------------------------------
    def setup_caches(self, max_batch_size: int, max_seq_length: Optional[int] = None, page_size: int = 16,
                     num_pages: Optional[int] = None) -> None:
        """``num_pages`` sizes every pool directly; else the pool holds
        ``max_batch_size`` requests of ``max_seq_length`` tokens (the reference's
        sizing rule, backends/base/engine.py:66-93, without its +1 page)."""
        if self.model is None:
            raise RuntimeError("load_model first")
        if num_pages is None:
            if max_seq_length is None:
                raise ValueError("give num_pages or max_seq_length")
            num_pages = max_batch_size * (-(-max_seq_length // page_size))
        self.page_size = page_size
        self.cache = CacheManager(self.model.cache_needs(), page_size, num_pages, max_batch_size, self.dtype,
                                  self.device)
        self.model.attach_caches(self.cache.layer_caches)
        self.runner = StepRunner(self.model, self.cache, self.model.spec.vocab_size, self.device)

    # -- the step function ---------------------------------------------------------
    def admit(self, req_id) -> None:
        self.cache.admit(req_id)

    def release(self, req_id) -> None:
        self.cache.release(req_id)

    @torch.inference_mode()
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        return self.runner.step(entries)
