"""Feed-forwards. SwiGLU as in the reference (engine/model.py:317-320):
down(silu(gate(x)) * up(x)), no biases; gate and up are one product here, and the
down projection takes the residual in its epilogue."""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, Part, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(Part):
    """params: hidden_size, intermediate_size. tensors: gate_proj/up_proj/down_proj .weight."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(spec.tensor_name("gate_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("up_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("down_proj.weight"), (hidden, inter), "matrix"),
        ]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.intermediate_size = int(spec.params["intermediate_size"])
        # Rows [0, I) are the gate, rows [I, 2I) the up projection.
        self.gate_up_weight = torch.cat(
            [tensors.pop(spec.tensor_name("gate_proj.weight")), tensors.pop(spec.tensor_name("up_proj.weight"))], dim=0
        ).contiguous()
        self.down_weight = tensors.pop(spec.tensor_name("down_proj.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        gate_up = ops.linear(x, self.gate_up_weight, None)
        return ops.linear(ops.silu_mul(gate_up), self.down_weight, None, residual)
