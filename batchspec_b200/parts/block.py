"""Pre-norm residual block (batchspec/models/base_model.py:53-56):
h = x + m mixer(norm1(x));  x' = h + m ffn(norm2(h)), m = ``residual_mult`` (1 unless the design scales its
branches).  The adds are carried as a pending branch output and fused into the following norm kernel; the residual
stream itself is float32.  A block returns its last branch unscaled; ``residual_mult`` is what whoever adds it
multiplies it by (the next block gets it as ``pending_scale``)."""
from __future__ import annotations

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, register_part


@register_part(BLOCKS, "prenorm")
class PreNormBlock(Block):
    SLOTS = {"norm1": NORMS, "mixer": MIXERS, "norm2": NORMS, "ffn": FEED_FORWARDS}

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0):
        a = self.norm1.forward(resid, pending, pending_scale)
        y = self.mixer.forward(a, ctx, cache)
        f = self.norm2.forward(resid, y, self.residual_mult)
        return resid, self.ffn.forward(f, ctx)


@register_part(BLOCKS, "prenorm_mixer")
class PreNormMixerBlock(Block):
    """A pre-norm layer without a feed-forward: x' = x + m mixer(norm1(x))."""
    SLOTS = {"norm1": NORMS, "mixer": MIXERS}

    def __init__(self, residual_mult: float = 1.0, **parts):
        super().__init__(**parts)
        self.residual_mult = float(residual_mult)

    def forward(self, resid, pending, ctx, cache, pending_scale: float = 1.0):
        a = self.norm1.forward(resid, pending, pending_scale)
        return resid, self.mixer.forward(a, ctx, cache)
