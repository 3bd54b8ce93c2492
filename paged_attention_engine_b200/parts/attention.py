"""Grouped-query attention over the paged cache (engine/model.py:284-315, engine/attention.py).

q, k and v are one fused projection with bias; q and k are rotated; the rotated k and v
go to the pages of this step's slots; every query attends the keys of its own request
at positions j <= p (and p - j < window when the layer has one), read in place through
the block table. Query head h reads kv head h // (heads / kv_heads)
(engine/attention.py:46-74); scores are scaled by `scale` (engine/model.py:59-62).
The output projection takes the residual in its epilogue.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, CacheNeed, Part, TensorSpec


@MIXERS.register("gqa_attention")
class GQAAttention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, scale, window,
    position_encoding (a dict with its `kind`, or None).
    tensors: q_proj/k_proj/v_proj .weight (+ .bias), o_proj.weight."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        p = spec.params
        hidden, d = int(p["hidden_size"]), int(p["head_dim"])
        nq, nkv = int(p["num_heads"]) * d, int(p["num_kv_heads"]) * d
        out = []
        for name, rows in (("q_proj", nq), ("k_proj", nkv), ("v_proj", nkv)):
            out.append(TensorSpec(spec.tensor_name(f"{name}.weight"), (rows, hidden), "matrix"))
            if p.get("qkv_bias", False):
                out.append(TensorSpec(spec.tensor_name(f"{name}.bias"), (rows,), "vector"))
        out.append(TensorSpec(spec.tensor_name("o_proj.weight"), (hidden, nq), "matrix"))
        return out

    @classmethod
    def sub_parts(cls, spec: PartSpec) -> list[tuple[str, PartSpec]]:
        enc = spec.params.get("position_encoding")
        if enc is None:
            return []
        return [("position_encoding", PartSpec(enc["kind"], {k: v for k, v in enc.items() if k != "kind"}, spec.prefix))]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        p = spec.params
        return CacheNeed(int(p["num_kv_heads"]), int(p["head_dim"]), int(p.get("window", 0)))

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = int(p.get("window", 0))
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"gqa_attention: {self.num_heads} heads over {self.num_kv_heads} kv heads")
        names = ("q_proj", "k_proj", "v_proj")
        # One projection for q | k | v: the rows are stacked in that order.
        self.qkv_weight = torch.cat([tensors.pop(spec.tensor_name(f"{n}.weight")) for n in names], dim=0).contiguous()
        self.qkv_bias = None
        if p.get("qkv_bias", False):
            self.qkv_bias = torch.cat([tensors.pop(spec.tensor_name(f"{n}.bias")) for n in names], dim=0).contiguous()
        self.o_weight = tensors.pop(spec.tensor_name("o_proj.weight"))
        built = self.build_sub_parts(tensors)
        self.position_encoding = built[0] if built else None

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        group = ctx.groups[cache.group]
        table = self.position_encoding.table(ctx) if self.position_encoding is not None else None
        slots = group.slots if cache.writes else None
        project = getattr(ops, "qkv_projection", None)
        if project is not None:          # the product, the rotation and the page write as one call
            qkv = project(x, self.qkv_weight, self.qkv_bias, table, slots, cache.keys, cache.values,
                          self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size)
        else:
            qkv = ops.rotary_qk_cache_write(
                ops.linear(x, self.qkv_weight, self.qkv_bias), table, slots, cache.keys, cache.values,
                self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size,
            )
        out = ops.paged_attention(
            qkv, cache.keys, cache.values, group.block_table, ctx.q_start, ctx.q_pos0, ctx.kv_len,
            self.num_heads, self.num_kv_heads, self.head_dim, cache.page_size,
            ctx.max_q_len, ctx.max_kv_len, self.scale, self.window, num_single=ctx.num_single,
            multi_index=getattr(ctx, "multi_index", None),
        )
        return ops.linear(out, self.o_weight, None, residual)
