"""Arrangements of a layer's parts. The reference's only one (engine/model.py:340-349):
norm, mixer, add; norm, feed-forward, add. The residual sum is made in 32-bit inside the
epilogue of each branch's last product."""

from __future__ import annotations

from .base import BLOCKS, Block


@BLOCKS.register("pre_norm_residual")
class PreNormResidual(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, ctx, hidden, layer, cache):
        # `hidden` may be a product that is still to be summed; the norm's kernel sums it, and
        # `materialized` then hands out the summed tensor without another launch.
        normed = layer.mixer_norm.forward(ctx, hidden)
        hidden = layer.mixer.forward(ctx, normed, ctx.ops.materialized(hidden), cache)
        normed = layer.feed_forward_norm.forward(ctx, hidden)
        return layer.feed_forward.forward(ctx, normed, ctx.ops.materialized(hidden))
