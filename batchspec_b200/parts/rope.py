"""Rotary position encoding part.

Frequencies: f_j = theta^(-2j/rotary_dim) (batchspec/models/modules/rope.py:27-31),
optionally rescaled by the llama3 rule whose constants the reference forwards
(rope.py:33-44) or divided by a plain factor (``rope_scale``).  The table is built
in float64 on the host and held as two float32 numbers per frequency; the kernels form
the angle position * f_j in float64 and reduce it to [-pi, pi] there, so that it is
right to 2e-7 rad at any position; sine, cosine and the rotation are float32.

Pairing: the reference rotates adjacent pairs after permuting Wq/Wk rows offline
(tools/prepare_model/convert_weights.py:112-128); this part keeps the
checkpoint's row order and rotates (j, j + rotary_dim/2), which gives the same
scores.  ``interleaved=True`` rotates adjacent pairs for checkpoints that were
permuted.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import POSITION_ENCODINGS, PositionEncoding, Runtime, register_part


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    j = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / rotary_dim)
    if scaling:
        kind = scaling["rope_type"]
        factor = float(scaling["factor"])
        if kind == "linear":
            f = f / factor
        elif kind == "llama3":
            low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
            old = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            smooth = ((old / wavelen) - low) / (high - low)
            mid = (1.0 - smooth) * f / factor + smooth * f
            f = torch.where(wavelen > old / low, f / factor, torch.where(wavelen < old / high, f, mid))
        else:
            raise ValueError(f"rope scaling {kind!r} is not supported")
    return f


@register_part(POSITION_ENCODINGS, "rope")
class RotaryEmbedding(PositionEncoding):
    graph_safe = True
    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling: Optional[dict] = None,
                 rotary_dim: Optional[int] = None, interleaved: bool = False):
        self.runtime = runtime
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        self.interleaved = bool(interleaved)
        self.frequencies = rope_inv_freq(self.rotary_dim, theta, scaling)            # float64, on the host
        self.inv_freq = ops.rope_frequency_table(self.frequencies, runtime.device)

    def rope_table(self):
        return self.inv_freq, self.rotary_dim, self.interleaved

    def apply(self, q, k, ctx):
        ops.rope_inplace(q, ctx.positions, self.inv_freq, self.rotary_dim, self.interleaved)
        ops.rope_inplace(k, ctx.positions, self.inv_freq, self.rotary_dim, self.interleaved)


@register_part(POSITION_ENCODINGS, "none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def apply(self, q, k, ctx):
        return None
