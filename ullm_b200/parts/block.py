"""Arrangement of a layer: pre-norm, residual stream.

ullm/models/qwen3.py:160-178: the stream is carried as (x, residual).  The
first block takes residual = x; afterwards each norm is the fused form
"residual <- x + residual (32-bit sum, rounded on store); h = norm(sum)".
"""

from __future__ import annotations

from .base import Block
from .registry import register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None):
        super().__init__()
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        n = names or {}
        self.names = {
            "mixer": n.get("mixer", "mixer."),
            "feed_forward": n.get("feed_forward", "feed_forward."),
            "mixer_norm": n.get("mixer_norm", "mixer_norm."),
            "feed_forward_norm": n.get("feed_forward_norm", "feed_forward_norm."),
        }

    def subparts(self):
        return {
            self.names["mixer_norm"]: self.mixer_norm,
            self.names["mixer"]: self.mixer,
            self.names["feed_forward_norm"]: self.feed_forward_norm,
            self.names["feed_forward"]: self.feed_forward,
        }

    def activation_elems(self):
        # the normed rows, and the wider of the two sub-layers (they run one after the other)
        size = getattr(self.mixer_norm, "size", 0)
        return size + max(self.mixer.activation_elems(), self.feed_forward.activation_elems())

    def forward(self, x, residual, ctx, cache):
        """x: the previous sub-layer's output (the embedding for the first
        block, with residual None).  Returns (feed-forward output, residual);
        the caller's final norm adds them."""
        T = x.shape[0]
        h = ctx.workspace.tokens("block.normed", T, x.shape[1], x.dtype)
        if residual is None:
            residual = x
            self.mixer_norm.forward(x, None, out=h)
        else:
            self.mixer_norm.forward(x, residual, out=h)
        a = self.mixer.forward(h, ctx, cache)
        self.feed_forward_norm.forward(a, residual, out=h)
        y = self.feed_forward.forward(h, ctx)
        return y, residual
