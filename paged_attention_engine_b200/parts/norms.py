"""Norms. RMSNorm as the reference computes it (engine/model.py:117-123): the mean of the
squares and the scaling in 32-bit, no bias, no mean subtraction. The kernel multiplies
by the weight in 32-bit too and rounds once; the reference rounds before and after the
weight, which costs one more rounding in bfloat16 and nothing in float32."""

from __future__ import annotations

from ..config.model_spec import PartSpec
from .base import NORMS, Part, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Part):
    """params: size, eps. tensors: weight [size]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["size"]),), "scale")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.weight = tensors[spec.tensor_name("weight")]

    def forward(self, ctx, x):
        return self.ops.rms_norm(x, self.weight, self.eps)
