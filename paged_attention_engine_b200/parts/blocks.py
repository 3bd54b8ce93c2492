"""Arrangements of a layer's parts. The reference's only one (engine/model.py:340-349):
norm, mixer, add; norm, feed-forward, add. The residual sum is made in 32-bit inside the
epilogue of each branch's last product."""

from __future__ import annotations

from .base import BLOCKS


@BLOCKS.register("pre_norm_residual")
class PreNormResidual:
    def forward(self, ctx, hidden, layer, cache):
        hidden = layer.mixer.forward(ctx, layer.mixer_norm.forward(ctx, hidden), hidden, cache)
        return layer.feed_forward.forward(ctx, layer.feed_forward_norm.forward(ctx, hidden), hidden)
