"""Rotary position encoding of the `default` type (engine/model.py:126-161).

inv_freq[i] = 1 / theta^(2i/d) is computed in float32 from an integer range, exactly
as the reference does (engine/model.py:132-135); the angle position x inv_freq and its
cosine and sine are float32 on the device, one table per step shared by every layer
that uses the same (head_dim, theta). Pairs are (j, j + d/2) (engine/model.py:126-129).
"""

from __future__ import annotations

import torch

from .base import POSITION_ENCODINGS, Part


@POSITION_ENCODINGS.register("rotary")
class Rotary(Part):
    """params: head_dim, theta. No tensors."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        if self.head_dim % 2:
            raise ValueError(f"rotary: head_dim {self.head_dim} must be even")
        exponent = torch.arange(0, self.head_dim, 2, dtype=torch.int64).to(torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (exponent / self.head_dim))).to(runtime.device)
        self._key = ("rotary", self.head_dim, self.theta)

    def table(self, ctx):
        """float32 [tokens, head_dim]: cosines in the first half of a row, sines in the second."""
        if self._key not in ctx.memo:
            ctx.memo[self._key] = self.ops.rotary_table(ctx.positions, self.inv_freq)
        return ctx.memo[self._key]
