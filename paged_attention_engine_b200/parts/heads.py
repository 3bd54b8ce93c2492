"""Token embedding (engine/model.py:401: a row gather, no scaling) and the language-model
head (engine/model.py:406: a product without bias at the wanted rows only; the head is the
embedding table itself when the checkpoint ties them, engine/model.py:220-222). Logits
leave the head in float32."""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import EMBEDDINGS, HEADS, Part, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: vocab_size, hidden_size. tensors: weight [vocab, hidden]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors[spec.tensor_name("weight")]

    def step_weight_bytes(self, num_tokens: int) -> int:
        """A step reads one row of the table per token, not the table. (When the head is tied to it,
        the head reads all of it and counts it.)"""
        return num_tokens * self.weight.shape[1] * self.weight.element_size()

    def forward(self, ctx):
        # A negative id is "the token sampled for this request in the step before" (see
        # StepContext.feedback); the kernel looks it up on the device.
        return self.ops.embedding(ctx.token_ids, self.weight, getattr(ctx, "feedback", None))


@HEADS.register("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied_to (a tensor's full name, or None).
    tensors: weight [vocab, hidden] unless tied."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        if spec.params.get("tied_to"):
            return []
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        tied = spec.params.get("tied_to")
        self.weight = tensors[tied] if tied else tensors[spec.tensor_name("weight")]

    def forward(self, ctx, rows):
        return self.ops.linear(rows, self.weight, None, None, out_dtype=torch.float32)
