"""Weights by tensor name: from a model folder, or drawn at random from a seed.

The reference loads one converted ``model.pth`` with ``strict=True``
(batchspec/backends/standard_engine.py:41-46) after an offline pass that renames,
permutes and fuses (tools/prepare_model/convert_weights.py:141-171).  Here the
folder's safetensors are read under their own names; fusing is each part's
``bind``.  Every problem of a folder is collected and raised once.

dtype rule: ``matrix`` tensors are held in the run dtype; ``vector`` tensors too,
except that in a bfloat16 run one that the file stores in 32-bit stays 32-bit;
``int`` tables become int32.  In a float32 run everything floating is float32.
"""
from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Dict, List, Optional

import torch

from ..parts.base import ParamSpec
from .safetensors_io import open_model_files, write_safetensors


class WeightsError(ValueError):
    """Lists every missing tensor, unexpected tensor and wrong shape of a folder."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_dtype=(), unequal=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        self.unequal = list(unequal)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + ", ".join(
                f"{n} is {got}" for n, got in self.wrong_dtype))
        if self.unequal:
            lines.append(f"  tensors that must be copies of another and are not ({len(self.unequal)}): " + ", ".join(
                f"{n} differs from {other}" for n, other in self.unequal))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _held_dtype(spec: ParamSpec, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int":
        return torch.int32
    if spec.role == "vector" and run_dtype != torch.float32 and stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def load_weights(model_dir, specs: Dict[str, ParamSpec], run_dtype: torch.dtype, device,
                 ignore_suffixes=(), ignore_names=(), must_equal: Optional[Dict[str, str]] = None) -> Dict[str, torch.Tensor]:
    """``must_equal``: name -> name of a wanted tensor.  Such a tensor may be absent; if the folder has it, it
    has to be an exact copy of the other one (a tied head stored a second time), else that is an error."""
    must_equal = dict(must_equal or {})
    files = open_model_files(model_dir)
    where: Dict[str, object] = {}
    for f in files:
        for name in f.entries:
            where[name] = f
    missing = [n for n in specs if n not in where]
    unexpected = [n for n in where if n not in specs and n not in ignore_names and n not in must_equal
                  and not any(n.endswith(s) for s in ignore_suffixes)]
    wrong_shape, wrong_dtype, unequal = [], [], []
    for name, other in must_equal.items():
        if name in where and other in where:
            a, b = where[name].tensor(name), where[other].tensor(other)
            if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
                unequal.append((name, other))
    for name, spec in specs.items():
        if name not in where:
            continue
        dtype, shape = where[name].entries[name]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((name, shape, spec.shape))
        if (spec.role == "int" and dtype not in _INTS) or (spec.role != "int" and dtype not in _FLOATS):
            wrong_dtype.append((name, str(dtype).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype or unequal:
        raise WeightsError(model_dir, missing, unexpected, wrong_shape, wrong_dtype, unequal)
    out = {}
    for name, spec in specs.items():
        t = where[name].tensor(name)
        out[name] = t.to(device=device, dtype=_held_dtype(spec, t.dtype, run_dtype)).contiguous()
    return out


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: ParamSpec, seed: int, std: float, norm_std: float,
                  device="cpu") -> torch.Tensor:
    """float32 draw for one tensor, a function of (seed, name) only, so the values
    do not depend on the order tensors are made in."""
    gen = torch.Generator(device=device)
    gen.manual_seed(_seed_for(seed, name))
    if spec.role == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    if spec.init == "ones_normal":
        return t.mul_(norm_std).add_(1.0)
    return t.mul_(std)


def random_weights(specs: Dict[str, ParamSpec], seed: int, run_dtype: torch.dtype, device,
                   std: float = 0.02, norm_std: float = 0.01, stored_dtype: Optional[torch.dtype] = None,
                   draw_on_device: bool = False) -> Dict[str, torch.Tensor]:
    """Random model in memory.  Drawn on the CPU (same values as a folder written by
    ``write_random_model`` with the same seed, after its rounding to
    ``stored_dtype``) unless ``draw_on_device``, which draws with the device's
    generator (other values, same distribution; for large benchmark models)."""
    out = {}
    for name, spec in specs.items():
        t = random_tensor(name, spec, seed, std, norm_std, device=device if draw_on_device else "cpu")
        if stored_dtype is not None and spec.role != "int":
            t = t.to(stored_dtype)
        out[name] = t.to(device=device, dtype=_held_dtype(spec, t.dtype, run_dtype)).contiguous()
    return out


def write_random_model(config, model_dir, seed: int, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, norm_std: float = 0.01) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` with weights
    drawn from ``seed``: matrices N(0, std), norm scales 1 + N(0, norm_std), stored
    as ``dtype``."""
    from ..config.model_config import save_config
    from ..models import get_model
    from ..parts.base import Runtime
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    save_config(config, model_dir)
    model = get_model(config, Runtime(torch.float32, torch.device("cpu")))
    specs = model.param_specs()
    write_safetensors(model_dir / "model.safetensors", (
        (name, random_tensor(name, spec, seed, std, norm_std).to(torch.int32 if spec.role == "int" else dtype))
        for name, spec in specs.items()))
    return model_dir
