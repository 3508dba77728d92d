"""Pre-norm residual block (batchspec/models/base_model.py:53-56):
h = x + mixer(norm1(x));  x' = h + ffn(norm2(h)).  The adds are carried as a
pending branch output and fused into the following norm kernel; the residual
stream itself is float32."""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, register_part


@register_part(BLOCKS, "prenorm")
class PreNormBlock(Block):
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "ffn": FEED_FORWARDS}

    def forward(self, resid, pending, ctx, cache):
        a = self.norm1.forward(resid, pending)
        y = self.mixer.forward(a, ctx, cache)
        f = self.norm2.forward(resid, y)
        return resid, self.ffn.forward(f, ctx)
