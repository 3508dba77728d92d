"""SwiGLU feed-forward part (batchspec/models/modules/feedforward.py:25-27,62):
u = x W13^T with W13 = [gate; up] fused at load (feedforward.py:35-38),
m = silu(u[:, :I]) * u[:, I:], out = m W2^T.  No biases.  In bfloat16 the fused matrix is stored with gate and up
rows interleaved in groups of 8 (8 gate rows, then their 8 up rows) and decode-sized steps apply the activation inside the product."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import FEED_FORWARDS, FeedForward, ParamSpec, Runtime, register_part


@register_part(FEED_FORWARDS, "swiglu")
class SwiGLU(FeedForward):
    graph_safe = True
    def __init__(self, runtime: Runtime, dim: int, intermediate: int):
        self.runtime, self.dim, self.intermediate = runtime, int(dim), int(intermediate)
        self.w13 = self.w2 = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"gate": ParamSpec((self.intermediate, self.dim)),
                "up": ParamSpec((self.intermediate, self.dim)),
                "down": ParamSpec((self.dim, self.intermediate))}

    def bind(self, params):
        # bfloat16: gate and up rows interleaved in groups, so that the GEMM's epilogue can apply the activation
        # (a CTA then holds matching gate and up outputs); float32: the reference's [gate; up] halves
        self.group = ops.GLU_GROUP if (self.runtime.dtype == torch.bfloat16
                                       and self.intermediate % ops.GLU_GROUP == 0) else 0
        if self.group:
            self.w13 = ops.interleave_gate_up(params["gate"], params["up"], self.group)
        else:
            self.w13 = torch.cat([params["gate"], params["up"]], dim=0).contiguous()
        self.w2 = params["down"].contiguous()

    def forward(self, x, ctx):
        if self.group:
            with bucket("mlp.gate_up_proj"):
                m = ops.linear_glu(x, self.w13, self.group)
        else:
            with bucket("mlp.gate_up_proj"):
                u = ops.linear(x, self.w13)
            m = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
            with bucket("mlp.act"):
                ops.silu_mul(u, m)
        with bucket("mlp.down_proj"):
            return ops.linear(m, self.w2)
