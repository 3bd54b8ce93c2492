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
        gate = tensors.pop(spec.tensor_name("gate_proj.weight"))
        up = tensors.pop(spec.tensor_name("up_proj.weight"))
        # Gate and up are one product. Where the kernels offer it, their rows alternate in
        # blocks (16 gate rows, their 16 up rows, ...) so that SiLU x up runs inside the
        # product; else rows [0, I) are the gate and rows [I, 2I) the up projection.
        interleave = getattr(self.ops, "interleave_gate_up", None)
        self.gate_up_weight = interleave(gate, up) if interleave is not None else None
        self.interleaved = self.gate_up_weight is not None
        if not self.interleaved:
            self.gate_up_weight = torch.cat([gate, up], dim=0).contiguous()
        self.down_weight = tensors.pop(spec.tensor_name("down_proj.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        if self.interleaved:
            hidden = ops.linear_swiglu(x, self.gate_up_weight)
        else:
            hidden = ops.silu_mul(ops.linear(x, self.gate_up_weight, None))
        return ops.linear(hidden, self.down_weight, None, residual)
