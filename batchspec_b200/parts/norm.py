"""RMSNorm part (batchspec/models/modules/normalization.py:24-39): float32
x * rsqrt(mean(x^2) + eps), cast to the run dtype, then times the weight.
Fused with the residual add that precedes it (base_model.py:53,56)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import NORMS, Norm, ParamSpec, Runtime, register_part


@register_part(NORMS, "rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    def __init__(self, runtime: Runtime, dim: int, eps: float):
        self.runtime, self.dim, self.eps = runtime, int(dim), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.dim,), role="vector", init="ones_normal")}

    def bind(self, params):
        self.weight = params["weight"]

    def forward(self, resid, delta=None):
        out = torch.empty(resid.shape, dtype=self.runtime.dtype, device=resid.device)
        with bucket("norm"):
            ops.add_rmsnorm(resid, delta, self.weight, self.eps, out)
        return out
