"""The decoder that runs: parts built from a `ModelSpec`, run in the schedule's order.

The reference writes its model once as a Python loop over identical layers
(engine/model.py:322-351). Here the loop runs over the schedule; each entry names a
layer (whose parts may differ from every other layer's) and the cache it reads and
writes. One call of `forward` is one traversal, counted in `forward_pass_count`
as the reference counts it (engine/model.py:180-186,338) so that a test can tell a
batched step from a loop over requests.
"""

from __future__ import annotations

import os
from typing import Any

import torch

from ..config.model_spec import ModelSpec
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, REGISTRIES, Runtime, layer_part_specs


# PAE_NVTX=1 marks every step's traversal and every schedule entry with an NVTX range, for a
# timeline profiler (the reference has no tracing at all; its stand-ins, the pass counter and the
# scheduler's event log, are kept as well).
NVTX = os.environ.get("PAE_NVTX", "0") not in ("", "0")


class Layer:
    """A layer as it runs: the block and the parts that the block kind declares, each under
    its role's name (`layer.mixer`, `layer.mixer_norm`, ...)."""

    def __init__(self, block: Any, parts: dict[str, Any]) -> None:
        self.block = block
        self.parts = parts
        for role, part in parts.items():
            setattr(self, role, part)


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.ops = runtime.ops
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, tensors, runtime)
        self.head = HEADS.get(spec.head.kind)(spec.head, tensors, runtime)
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, tensors, runtime)
        self.layers: list[Layer] = []
        for layer in spec.layers:
            built = {
                role: REGISTRIES[registry].get(part.kind)(part, tensors, runtime)
                for role, registry, part in layer_part_specs(layer)
            }
            self.layers.append(Layer(BLOCKS.get(layer.block)(), built))
        self.forward_pass_count = 0
        self.graph_safe = all(getattr(part, "graph_safe", True) for part in self.parts())

    def parts(self) -> list[Any]:
        """Every part of the model, blocks included (parts nested inside others are theirs)."""
        out = [self.embedding, self.head, self.final_norm]
        for layer in self.layers:
            out += [layer.block, *layer.parts.values()]
        return out

    def forward(self, ctx, entry_caches) -> torch.Tensor | None:
        """Runs the step's tokens through every schedule entry; float32 logits
        [wanted, vocab] at `ctx.logit_rows`, or None when nothing is wanted."""
        self.forward_pass_count += 1
        if NVTX:
            torch.cuda.nvtx.range_push(f"traversal: {ctx.num_tokens} tokens of {ctx.num_seqs} requests")
        hidden = self.embedding.forward(ctx)
        for position, entry in enumerate(self.spec.schedule):
            layer = self.layers[entry.layer]
            if NVTX:
                torch.cuda.nvtx.range_push(f"entry {position}: layer {entry.layer}")
            hidden = layer.block.forward(ctx, hidden, layer, entry_caches[position])
            if NVTX:
                torch.cuda.nvtx.range_pop()
        if NVTX:
            torch.cuda.nvtx.range_pop()
        if ctx.logit_rows.numel() == 0:
            return None
        # A step that wants the logits of all its tokens (decoding) needs no gather, and the final
        # norm can finish the last product itself.
        rows = hidden if getattr(ctx, "wants_every_token", False) else self.ops.gather_rows(hidden, ctx.logit_rows)
        # The head's product may still be waiting for its sum (a step of few wanted rows): logits leave as a tensor.
        return self.ops.materialized(self.head.forward(ctx, self.final_norm.forward(ctx, rows)))
