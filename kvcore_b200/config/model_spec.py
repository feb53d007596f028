"""Architecture-neutral description of a decoder: what each layer is made of, and in
which order layers run.

A ``ModelSpec`` is plain data.  An architecture's config parser (for example
``kvcore_b200.config.llama``) turns the keys of config.json into one; the model builder
(``kvcore_b200.parts.model.build_model``) turns it into parts by looking up each
``PartSpec.kind`` in the part registries.  Nothing here knows a model family.

* ``PartSpec(kind, params)`` names a registered part and the constants it is built with.
* ``LayerSpec`` holds the parts of one layer (mixer, feed-forward, norms) and the kind
  of block that arranges them, plus the prefix of its tensor names.
* ``ScheduleEntry(layer, cache_of)`` is one run of a layer.  The schedule is a list, so a
  layer may be named twice (shared weights; each run gets a cache of its own), and an
  entry may set ``cache_of`` to the index of an earlier *entry* to read that entry's
  cache instead of writing one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


def _freeze(params: Mapping[str, Any] | None) -> Mapping[str, Any]:
    return MappingProxyType(dict(params or {}))


@dataclass(frozen=True)
class PartSpec:
    """A registered part kind and the constants handed to its constructor."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", _freeze(self.params))

    def with_params(self, **updates: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(updates)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer, a feed-forward and its norms."""

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "norms", MappingProxyType(dict(self.norms)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of ``layers[layer]``; ``cache_of`` names an earlier entry whose cache is read."""

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the builder needs: sizes, parts, run order and generation constants."""

    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    embedding: PartSpec
    final_norm: PartSpec
    lm_head: PartSpec
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    stored_dtype: str | None = None

    def __post_init__(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("a model needs a non-empty layer schedule")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(
                    f"schedule[{index}] names layer {entry.layer}, "
                    f"but the model has {len(self.layers)} layers"
                )
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ValueError(
                        f"schedule[{index}].cache_of={entry.cache_of} must name an earlier entry"
                    )
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(
                        f"schedule[{index}].cache_of={entry.cache_of} names an entry that "
                        "itself borrows a cache; name the owner instead"
                    )


def default_schedule(num_layers: int) -> tuple[ScheduleEntry, ...]:
    """Each layer once, in order, each with a cache of its own."""
    return tuple(ScheduleEntry(layer=i) for i in range(num_layers))


__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "ScheduleEntry", "default_schedule"]
