"""Interfaces and registries of the parts a layer is put together from.

A part is built from its `PartSpec` (sizes and constants as parameters) and from
its tensors; it runs on the flattened batch of one step through the kernels in
`ctx.ops`. Five registries hold the part classes by name: mixers, feed-forwards,
norms, position encodings and blocks (the arrangement of the others in a layer),
plus embeddings and heads. Registering a class under a new name is all it takes to
make a new part usable from a `ModelSpec`; nothing in the cache manager, the step
function or the scheduler has to change.

What each kind of part must provide:

  every part    `tensor_specs(spec)`: the tensors it reads from the checkpoint
                (full names, shapes, kind), used by the loader's validation and by
                the random-weights mode; `__init__(spec, tensors, runtime)`;
                `sub_parts(spec)`: the parts it holds inside itself (an attention's
                position encoding), as (registry name, PartSpec) pairs: the loader
                and the random-weights mode follow them, so a part with parts of
                its own needs no line anywhere else.
  norm          `forward(ctx, x) -> y`, same shape.
  position enc. `table(ctx)`: whatever its mixers need for this step's positions,
                computed once per step and memoised in `ctx.memo`.
  mixer         `cache_need(spec)`: None, or a `CacheNeed` (kv heads, head size,
                window) that makes the cache manager give its schedule entry pages;
                `state_need(spec)`: None, or a `StateNeed` (shape per request) that
                makes the cache manager give it a fixed-size slot per request;
                `forward(ctx, x, residual, cache) -> residual + mixer(x)` where
                `cache` is the `EntryCache` of the schedule entry that runs.
  feed-forward  `forward(ctx, x, residual) -> residual + ff(x)`.
  block         `roles`: which parts a layer of this kind has and the registry each
                comes from ({"mixer_norm": "norm", "mixer": "mixer", ...}); the
                model builds exactly these from the `LayerSpec` and hands them to
                `forward(ctx, hidden, layer, cache) -> hidden` as attributes of
                `layer`. A block with other parts (four norms, one norm shared by two
                branches) declares other roles; nothing outside its class changes.

A part whose forward() looks at the step's host-side fields declares `graph_safe = False`.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Optional

import torch

from ..config.model_spec import PartSpec


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor. `kind` decides its storage and its random initialisation:

    matrix   a weight of a matrix product: engine dtype (bfloat16 or float32);
             drawn N(0, 0.02).
    vector   a bias: held in float32; drawn N(0, 0.02).
    scale    a norm's weight: held in float32; drawn 1 + N(0, 0.02).
    index    an integer table: held as int32; drawn uniformly from [0, shape[0]).
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values of a mixer: `window` 0 keeps all of them, w > 0 the last w."""

    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size, zeroed when the request is admitted."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class EntryCache:
    """What one schedule entry sees of the cache during a step."""

    group: int = -1                          # index of its page group, -1 without pages
    keys: Optional[torch.Tensor] = None      # [pages, kv_heads, page_size, head_dim]
    values: Optional[torch.Tensor] = None
    page_size: int = 0
    writes: bool = True                      # False when it reads another entry's cache
    state: Optional[torch.Tensor] = None     # [slots, *StateNeed.shape]


@dataclass
class Runtime:
    """What a part gets at construction: the kernels, the engine dtype and the device."""

    ops: Any
    dtype: torch.dtype
    device: torch.device


class Part:
    # A step that only decodes is recorded once as a CUDA graph and replayed. That is sound
    # for a part whose forward() depends on the step only through device tensors of `ctx`
    # (and its batch size). A part that reads the step's host-side fields (`host_q_lens`,
    # `host_state_slots`, ...) or branches on values sets this to False; a model that holds
    # such a part always runs eagerly.
    graph_safe = True

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return []

    @classmethod
    def sub_parts(cls, spec: PartSpec) -> list[tuple[str, PartSpec]]:
        """(registry name, PartSpec) of every part that this part builds inside itself."""
        return []

    def __init__(self, spec: PartSpec, tensors: dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.spec = spec
        self.runtime = runtime
        self.ops = runtime.ops

    def build_sub_parts(self, tensors: dict[str, torch.Tensor]) -> list[Any]:
        """The parts of `sub_parts`, built, in its order."""
        return [REGISTRIES[registry].get(sub.kind)(sub, tensors, self.runtime)
                for registry, sub in self.sub_parts(self.spec)]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed | None:
        return None

    @classmethod
    def state_need(cls, spec: PartSpec) -> StateNeed | None:
        return None


class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._classes: dict[str, type] = {}

    def register(self, name: str) -> Callable[[type], type]:
        def put(cls: type) -> type:
            self._classes[name] = cls
            return cls

        return put

    def get(self, name: str) -> type:
        if name not in self._classes:
            raise KeyError(f"no {self.what} is registered as '{name}'; known: {', '.join(sorted(self._classes))}")
        return self._classes[name]

    def names(self) -> list[str]:
        return sorted(self._classes)


class Block:
    """Arrangement of a layer's parts. `roles` maps each part's name in the layer to the
    name of the registry it comes from."""

    graph_safe = True
    roles: dict[str, str] = {}

    def forward(self, ctx, hidden, layer, cache):
        raise NotImplementedError


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

REGISTRIES: dict[str, Registry] = {
    "mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position_encoding": POSITION_ENCODINGS,
    "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS,
}


def layer_part_specs(layer) -> list[tuple[str, str, PartSpec]]:
    """(role, registry name, PartSpec) for every part of a `LayerSpec`, in the order in which its
    block kind declares them; raises when the layer lacks a declared role or has an undeclared one."""
    block = BLOCKS.get(layer.block)
    roles = getattr(block, "roles", None)
    if not roles:
        raise ValueError(f"block '{layer.block}' declares no roles (a dict: part name -> registry name)")
    missing = [r for r in roles if r not in layer.parts]
    extra = [r for r in layer.parts if r not in roles]
    if missing or extra:
        raise ValueError(
            f"a '{layer.block}' layer has the parts {', '.join(roles)}; "
            + (f"missing: {', '.join(missing)}; " if missing else "")
            + (f"not declared by the block: {', '.join(extra)}" if extra else "")
        )
    for role, registry in roles.items():
        if registry not in REGISTRIES:
            raise ValueError(f"block '{layer.block}': role '{role}' names the registry '{registry}'; known: {', '.join(REGISTRIES)}")
    return [(role, registry, layer.parts[role]) for role, registry in roles.items()]


def with_sub_parts(registry: str, spec: PartSpec) -> list[tuple[str, PartSpec]]:
    """(registry name, PartSpec) of a part and of every part nested inside it, outermost first."""
    out = [(registry, spec)]
    cls = REGISTRIES[registry].get(spec.kind)
    for sub_registry, sub in getattr(cls, "sub_parts", lambda _spec: [])(spec):
        out += with_sub_parts(sub_registry, sub)
    return out
