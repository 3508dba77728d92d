"""Grouped-query softmax attention over the paged cache
(batchspec/models/modules/attention/standard.py:51-73, attention/base.py:32-39,92-93).

Order, as in the reference: fused QKV projection; split into q [n,Hq,hd],
k [n,Hkv,hd], v [n,Hkv,hd]; position encoding on q and k; k and v written to
their cache pages (modules/kv_cache.py:64-83); causal attention of the new
queries over all cached keys of their request, scores scaled by 1/sqrt(hd) unless
a scale is given (standard_engine.py:132-143 passes none), query head h reading
kv head h // (Hq/Hkv); output projection.  An optional ``window`` keeps only the
last ``window`` keys (not a Llama option; the cache then asks for windowed pages).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import (MIXERS, POSITION_ENCODINGS, CacheSpec, Mixer, ParamSpec, PartSpec, Runtime, build_part,
                   register_part)


@register_part(MIXERS, "attention")
class Attention(Mixer):
    graph_safe = True
    def __init__(self, runtime: Runtime, dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position: PartSpec, window: Optional[int] = None, scale: Optional[float] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"attention kernels take head_dim in steps of 16 up to 256, got {head_dim}")
        self.runtime = runtime
        self.dim, self.n_heads, self.n_kv_heads, self.head_dim = int(dim), int(n_heads), int(n_kv_heads), int(head_dim)
        self.window = int(window) if window else 0
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part(POSITION_ENCODINGS, position, runtime)
        self.wqkv = self.wo = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        return {"q": ParamSpec((q, self.dim)), "k": ParamSpec((kv, self.dim)), "v": ParamSpec((kv, self.dim)),
                "o": ParamSpec((self.dim, q))}

    def bind(self, params):
        # rows [Wq; Wk; Wv], the reference's fusion order (attention/base.py:66-70)
        self.wqkv = torch.cat([params["q"], params["k"], params["v"]], dim=0).contiguous()
        self.wo = params["o"].contiguous()

    def cache_spec(self) -> CacheSpec:
        if self.window:
            return CacheSpec("window", (self.n_kv_heads, self.head_dim), self.window)
        return CacheSpec("full", (self.n_kv_heads, self.head_dim))

    def forward(self, x, ctx, cache):
        n = x.shape[0]
        Hq, Hkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        tables = ctx.tables[cache.group]
        table = self.position.rope_table()
        qkv = None
        if table is not None:
            # decode-sized bfloat16 steps with heads of 128: one kernel projects, rotates and appends to the cache
            with bucket("attn.qkv_proj"):
                qkv = ops.linear_qkv_rope(x, self.wqkv, Hq, Hkv, hd, table[0], table[1], table[2], ctx.positions,
                                          ctx.tok_entry, tables.kv_indptr, tables.kv_indices, cache.kv,
                                          tables.page_size, write_kv=cache.owner)
        if qkv is None:
            with bucket("attn.qkv_proj"):
                qkv = ops.linear(x, self.wqkv)
            if table is None:
                q = qkv[:, :Hq * hd].view(n, Hq, hd)
                k = qkv[:, Hq * hd:(Hq + Hkv) * hd].view(n, Hkv, hd)
                self.position.apply(q, k, ctx)
                inv_freq, rotary_dim, interleaved = None, 0, False
            else:
                inv_freq, rotary_dim, interleaved = table
            with bucket("attn.rope"):
                ops.rope_kv_append(qkv, Hq, Hkv, hd, inv_freq, rotary_dim, interleaved, ctx.positions, ctx.tok_entry,
                                   tables.kv_indptr, tables.kv_indices, cache.kv, tables.page_size,
                                   write_kv=cache.owner)
        out = torch.empty((n, Hq * hd), dtype=x.dtype, device=x.device)
        with bucket("attn.compute"):
            ops.paged_attention(qkv, out, cache.kv, ctx, tables, Hq, Hkv, hd, self.scale, self.window)
        with bucket("attn.o_proj"):
            return ops.linear(out, self.wo)
