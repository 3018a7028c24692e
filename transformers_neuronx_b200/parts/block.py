"""The arrangement of a layer's parts.

pre_norm  (src/transformers_neuronx/opt/model.py:336-376):  x += mixer(norm1(x)); x += ff(norm2(x))
post_norm (the reference rejects it, opt/config.py:23-24; this is the usual order):
                                                          x = norm1(x + mixer(x)); x = norm2(x + ff(x))

`x` is the 32-bit residual stream and is updated in place; `x_act` is its copy in the activation
type, which a block that feeds x itself into a matrix product needs on entry
(``needs_act_input``) and keeps current (``keeps_act_current``).
"""
from __future__ import annotations

from .base import NormedInput
from .registry import register_block


class PreNormBlock:
    needs_act_input = False
    keeps_act_current = False

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    @staticmethod
    def _normed(ctx, x, norm, part):
        """norm(x) as the part's input: for one token and a part that takes it, the norm is handed on
        to be applied inside the part's first product; otherwise its own kernel runs here."""
        fused = getattr(norm, "fused_params", None)
        if (x.shape[0] == 1 and ctx.act_dtype != x.dtype and getattr(part, "takes_normed_input", False)
                and fused is not None and fused() is not None):
            return NormedInput(ctx, x, norm)
        h = ctx.scratch(x.shape[0], x.shape[1])
        norm.forward(ctx, x, out_act=h)
        return h

    def forward(self, ctx, x, x_act):
        self.mixer.forward(ctx, self._normed(ctx, x, self.norm1, self.mixer), x)
        self.feed_forward.forward(ctx, self._normed(ctx, x, self.norm2, self.feed_forward), x)


class PostNormBlock:
    needs_act_input = True
    keeps_act_current = True

    def __init__(self, norm1, mixer, norm2, feed_forward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def forward(self, ctx, x, x_act):
        self.mixer.forward(ctx, x_act, x)
        self.norm1.forward(ctx, x, out_f32=x, out_act=x_act)      # in place: a row is read whole first
        self.feed_forward.forward(ctx, x_act, x)
        self.norm2.forward(ctx, x, out_f32=x, out_act=x_act)


register_block("pre_norm", PreNormBlock)
register_block("post_norm", PostNormBlock)
