"""Interfaces of the parts a layer is assembled from, and the registries that map a
``PartSpec.kind`` to a constructor.

Every part is built from plain numbers (its spec's params) plus ``dtype`` and ``device``;
none knows the model it sits in.  What each kind must provide:

* **Norm**: ``forward(x) -> y`` and ``forward_residual(h, residual) -> (y, residual)`` where
  ``residual`` is updated in place to ``h + residual`` and ``y = norm(residual)``.
* **PositionEncoding**: ``apply(q, k, ctx)`` rotating/shifting ``q [T,H,D]`` and ``k [T,KVH,D]``
  in place for the tokens of this step (``ctx.positions``).
* **Mixer**: ``forward(x [T,E], ctx, cache) -> [T,E]``.  It declares what it needs cached
  through ``cache_spec()`` (paged keys/values; ``None`` if none) and ``state_spec()`` (a
  fixed-size per-request state; ``None`` if none).  ``cache`` is the ``LayerCache`` of the
  schedule entry being run.
* **FeedForward**: ``forward(x [T,E], ctx) -> [T,E]``.
* **Block**: ``forward(h, residual, ctx, cache) -> (h, residual)``; arranges norms, mixer and
  feed-forward.  ``residual`` is ``None`` before the first block.

All parts expose their tensors to the loader through ``weight_slots()``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Iterable, Protocol

import torch

from ..config.model_spec import PartSpec


@dataclass
class WeightSlot:
    """One tensor of a checkpoint and where it goes.

    ``dest`` is the destination storage: a whole parameter, or a row-slice of a packed one
    (q/k/v rows of one projection matrix), or a strided view that scatters the tensor's rows
    (gate rows into every other run of 8 rows); in the last case ``file_shape`` is the shape
    the checkpoint stores and ``dest`` has the same number of elements in the same order.
    ``init`` tells the random-weights mode how to
    fill it ("normal", "ones", "zeros").  ``keep_f32`` lets a tensor that the file stores in
    32-bit stay 32-bit in a bfloat16 model: the loader then calls ``rebind`` with the
    32-bit tensor instead of casting into ``dest``.
    """

    name: str
    dest: torch.Tensor
    init: str = "normal"
    keep_f32: bool = False
    rebind: Callable[[torch.Tensor], None] | None = None
    file_shape: tuple[int, ...] | None = None

    @property
    def shape(self) -> tuple[int, ...]:
        """Shape of the tensor in a checkpoint."""
        return tuple(self.file_shape) if self.file_shape is not None else tuple(self.dest.shape)


@dataclass(frozen=True)
class CacheSpec:
    """Paged key/value needs of a mixer: entries with equal specs share a page group.

    ``window`` is ``None`` when every key stays visible, else the number of trailing keys a
    query sees; pages wholly behind the window are handed back while the request lives.
    """

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state of a mixer: one ``shape``-d tensor per live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    """Base of everything that may hold weights.

    ``graph_safe``: the part's forward launches the same kernels with the same host-side
    arguments for every batch of a given shape and reads batch contents only from device
    memory, so a decode step containing it may be captured in a CUDA graph and replayed.
    A part that branches on host copies of the batch (``ctx.host_*``) must leave it False.
    """

    graph_safe = False

    def weight_slots(self) -> list[WeightSlot]:
        return []

    def finalize_weights(self) -> None:
        """Called once after all slots are filled (repack, build derived tables)."""


class Summed:
    """Stands where a sub-layer's output would stand in the ``(h, residual)`` pair that runs through
    the blocks, when that output has already been added into ``residual``.  ``sumsq`` ``[T, pieces]``
    holds the squares of the rows of ``residual`` (for the norm that follows), or is None."""

    __slots__ = ("sumsq",)

    def __init__(self, sumsq: torch.Tensor | None) -> None:
        self.sumsq = sumsq


class Norm(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_residual(
        self, h: torch.Tensor, residual: torch.Tensor
    ) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def as_rms_scale(self) -> tuple[torch.Tensor, float] | None:
        """``(weight, eps)`` if this norm is exactly ``weight * x * rsqrt(mean(x^2) + eps)``, so that
        the part behind it may fold it into its first matrix product; ``None`` otherwise."""
        return None


class PositionEncoding(Part):
    def apply(self, q: torch.Tensor, k: torch.Tensor | None, ctx: Any) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_spec(self) -> CacheSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    # Optional: ``forward_prenorm(h, residual, rms_scale, ctx, cache) -> (out, residual)`` takes the
    # sub-layer input before its norm (``h`` a tensor or ``Summed``, ``residual`` a tensor or None)
    # together with the norm's ``as_rms_scale()``; it returns the sub-layer's output (a tensor, or
    # ``Summed`` if it has added it into the residual already) and the residual.  The block uses it
    # when both the norm and the part offer it.  (The same holds for a FeedForward, without ``cache``.)

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(
        self, h: torch.Tensor, residual: torch.Tensor | None, ctx: Any, cache: Any
    ) -> tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError


class PartFactory(Protocol):
    def __call__(self, *, dtype: torch.dtype, device: torch.device, **params: Any) -> Part: ...


class PartRegistry:
    """Kind name -> constructor, for one family of parts."""

    def __init__(self, family: str) -> None:
        self.family = family
        self._factories: dict[str, PartFactory] = {}

    def register(self, kind: str, factory: PartFactory | None = None, *, replace: bool = False):
        """Register ``factory`` under ``kind``; usable as a decorator."""

        def _add(target: PartFactory) -> PartFactory:
            if kind in self._factories and not replace:
                raise ValueError(f"{self.family} kind {kind!r} is already registered")
            self._factories[kind] = target
            return target

        return _add if factory is None else _add(factory)

    def unregister(self, kind: str) -> None:
        self._factories.pop(kind, None)

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._factories))

    def build(self, spec: PartSpec, *, dtype: torch.dtype, device: torch.device, **extra: Any) -> Part:
        if spec.kind not in self._factories:
            raise KeyError(
                f"unknown {self.family} kind {spec.kind!r}; registered: {', '.join(self.kinds())}"
            )
        params = dict(spec.params)
        params.update(extra)
        return self._factories[spec.kind](dtype=dtype, device=device, **params)


NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
BLOCKS = PartRegistry("block")
EMBEDDINGS = PartRegistry("embedding")
LM_HEADS = PartRegistry("lm head")


def collect_slots(parts: Iterable[Part]) -> list[WeightSlot]:
    slots: list[WeightSlot] = []
    for part in parts:
        slots.extend(part.weight_slots())
    return slots


__all__ = [
    "BLOCKS",
    "Block",
    "CacheSpec",
    "EMBEDDINGS",
    "FEED_FORWARDS",
    "FeedForward",
    "LM_HEADS",
    "MIXERS",
    "Mixer",
    "NORMS",
    "Norm",
    "POSITION_ENCODINGS",
    "Part",
    "PartRegistry",
    "PositionEncoding",
    "StateSpec",
    "WeightSlot",
    "collect_slots",
]
