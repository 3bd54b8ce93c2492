"""Architecture-neutral description of a decoder: which parts, with which constants,
in which order.

An architecture's builder (see `registry.py`) turns its typed configuration into a
`ModelSpec`. Everything after that (weight loading, random weights, the cache
manager, the model that runs) reads only the spec, so a new architecture is a new
builder and, if it needs them, new parts; nothing else changes.

A part is named by its registry key (`kind`) and carries its sizes and constants
as `params`; no part knows which model it is in. Layers may differ from one
another in every part, and in which parts they have: a layer is a block kind plus
the parts that this kind declares, by role. The order in which layers run is the `schedule`: a list
of entries that may name a layer twice (its weights are then shared, each run has
a cache of its own) or let an entry read the cache that an earlier entry wrote.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: registry key, constants, and where its tensors are in the checkpoint.

    `prefix` is put before the part's own tensor names ("q_proj.weight" becomes
    "model.layers.3.self_attn.q_proj.weight"); `names` renames single tensors
    for a checkpoint that calls them otherwise.
    """

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""
    names: Mapping[str, str] = field(default_factory=dict)

    def tensor_name(self, own_name: str) -> str:
        if own_name in self.names:
            return self.names[own_name]
        return f"{self.prefix}.{own_name}" if self.prefix else own_name


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block kind and the parts it arranges, by role.

    Which roles a layer has, and from which registry each part comes, is the block
    kind's own declaration (`roles` of the class registered under `block`): the usual
    decoder block has `mixer_norm`, `mixer`, `feed_forward_norm` and `feed_forward`;
    a block with four norms or one shared norm names its roles otherwise and nothing
    outside that class changes. `layer.mixer` reads `layer.parts["mixer"]`.
    """

    block: str
    parts: Mapping[str, PartSpec]

    def __getattr__(self, role: str) -> PartSpec:
        parts = object.__getattribute__(self, "parts")
        if role in parts:
            return parts[role]
        raise AttributeError(f"a '{object.__getattribute__(self, 'block')}' layer has no part '{role}'; it has: {', '.join(parts)}")


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. `cache_from` is the index of an EARLIER schedule entry whose
    keys and values this run reads instead of writing its own."""

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec

    def __post_init__(self) -> None:
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{pos}] names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < pos:
                    raise ValueError(
                        f"schedule[{pos}] reads the cache of entry {entry.cache_from}, which does not run before it"
                    )
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule[{pos}] reads the cache of entry {entry.cache_from}, which has none of its own"
                    )
