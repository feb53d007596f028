"""Interfaces of the parts a layer is assembled from, and the registries that map a
``PartSpec.kind`` to a constructor.

Every part is built from plain numbers (its spec's params) plus ``dtype`` and ``device``;
none knows the model it sits in.  What each kind must provide:

* **Norm**: ``forward(x) -> y`` and ``forward_residual(h, residual) -> (y, residual)`` where
  ``residual`` is updated in place to ``h + residual`` and ``y = norm(residual)``.
* **PositionEncoding**: ``apply(q, k, ctx)`` rotating/shifting ``q [T,H,D]`` and ``k [T,KVH,D]``
  in place for the tokens of this step (``ctx.positions``).
* **Mixer**: ``forward(x [T,E], ctx, cache) -> [T,E]``.  It declares what it needs cached
  through ``cache_spec()`` (what it keeps per cached token, in pages; ``None`` if nothing) and ``state_spec()`` (a
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
    """Paged needs of a mixer: what it keeps per cached token.  Entries with equal specs share a
    page group (one pool of page ids, one block table).

    A page of the group holds ``page_size`` tokens in each of ``planes`` tensors of shape
    ``[heads, page_size, width]``: keys and values of grouped-query attention are two planes of
    ``kv_heads`` heads of ``head_dim`` (``CacheSpec.keys_and_values``); a mixer that caches one
    vector per token declares one plane of one head.  ``window`` is ``None`` when every cached
    token stays visible, else the number of trailing tokens a query sees; pages wholly behind the
    window are handed back while the request lives.
    """

    planes: int
    heads: int
    width: int
    window: int | None = None

    def __post_init__(self) -> None:
        if self.planes <= 0 or self.heads <= 0 or self.width <= 0:
            raise ValueError(f"a cache spec needs positive planes, heads and width, got {self}")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive when set, got {self.window}")

    @classmethod
    def keys_and_values(cls, num_kv_heads: int, head_dim: int, window: int | None = None) -> "CacheSpec":
        return cls(2, int(num_kv_heads), int(head_dim), window)

    @property
    def elements_per_token(self) -> int:
        return self.planes * self.heads * self.width


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

    def ignorable_tensor_names(self) -> list[str]:
        """Names a checkpoint may carry for this part without a slot to load them into (buffers the
        part derives itself, a tied matrix stored twice).  A part that holds other parts adds theirs."""
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

    def cos_sin(self, ctx: Any) -> torch.Tensor | None:
        """Capability: an encoding that is a half-rotation of each head by per-token angles may return
        their ``[T, D/2, 2]`` 32-bit (cos, sin) table for this step's tokens; a mixer then fuses the
        rotation with its cache write (and, for decode steps, with its attention kernel) instead of
        calling ``apply``.  ``None`` (the default): the encoding is applied through ``apply``."""
        return None


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
