"""Rotary position encoding (half-rotation layout) with llama3 frequency scaling.

Rotation as the reference applies it (kvcore/model/layer/rotary_embedding.py:10-35, 92-127):
``inv_freq[j] = theta^(-2j/D)``, angle ``pos * inv_freq[j]`` in 32-bit, and for each head
``x' = x*cos + rotate_half(x)*sin`` with ``rotate_half(x) = cat(-x[D/2:], x[:D/2])``.

The frequency table is built once on the host in 64-bit and stored in 32-bit.  The
reference's rotary layer reads only the base; the ``llama3`` rule added here rescales each
frequency by its wavelength ``w = 2*pi/inv_freq`` against the original context length P:
kept when ``w < P/high``, divided by ``factor`` when ``w > P/low``, and blended linearly in
between with ``s = (P/w - low)/(high - low)``.  ``linear`` divides every frequency by ``factor``.
"""
from __future__ import annotations

import math

import torch

from .. import kernels as K
from .base import POSITION_ENCODINGS, PositionEncoding


def rope_inverse_frequencies(
    head_dim: int,
    theta: float,
    rope_type: str = "default",
    factor: float = 1.0,
    low_freq_factor: float = 1.0,
    high_freq_factor: float = 4.0,
    original_max_position_embeddings: int = 8192,
) -> torch.Tensor:
    """The ``[head_dim/2]`` table of rotation frequencies, 32-bit, on the CPU."""
    half = head_dim // 2
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float64)[:half] / head_dim
    inv_freq = 1.0 / (float(theta) ** exponents)
    if rope_type in (None, "default"):
        pass
    elif rope_type == "linear":
        inv_freq = inv_freq / float(factor)
    elif rope_type == "llama3":
        original = float(original_max_position_embeddings)
        low_wavelen = original / float(low_freq_factor)
        high_wavelen = original / float(high_freq_factor)
        wavelen = 2.0 * math.pi / inv_freq
        smooth = (original / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
        blended = (1.0 - smooth) * inv_freq / factor + smooth * inv_freq
        scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
        middle = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
        inv_freq = torch.where(middle, blended, scaled)
    else:
        raise ValueError(f"unsupported rope_type {rope_type!r}")
    return inv_freq.to(torch.float32)


class RotaryEncoding(PositionEncoding):
    """Holds the frequency table; the attention mixer fuses its rotation with the cache write."""

    graph_safe = True

    def __init__(
        self,
        *,
        head_dim: int,
        theta: float,
        rope_type: str = "default",
        factor: float = 1.0,
        low_freq_factor: float = 1.0,
        high_freq_factor: float = 4.0,
        original_max_position_embeddings: int = 8192,
        name: str | None = None,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.name = name
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {head_dim}")
        self.head_dim = int(head_dim)
        # layers with the same frequency parameters share one cos/sin table per step
        self.table_key = ("rope", int(head_dim), float(theta), str(rope_type), float(factor),
                          float(low_freq_factor), float(high_freq_factor), int(original_max_position_embeddings))
        table = rope_inverse_frequencies(
            head_dim, theta, rope_type, factor, low_freq_factor, high_freq_factor,
            original_max_position_embeddings,
        )
        self.inv_freq = table if torch.device(device).type == "meta" else table.to(device)

    def ignorable_tensor_names(self) -> list[str]:
        # checkpoints written from modules that register the frequency table as a buffer carry it;
        # the table is derived from the configuration here
        return [] if self.name is None else [f"{self.name}.inv_freq"]

    def cos_sin(self, ctx) -> torch.Tensor:
        """``[T, D/2, 2]`` (cos, sin) of this step's positions; one table per step and frequency table."""
        return ctx.shared(self.table_key, lambda: K.rope_table(ctx.positions, self.inv_freq))

    def apply(self, q: torch.Tensor, k: torch.Tensor | None, ctx) -> None:
        K.rope_inplace(q, k, ctx.positions, self.inv_freq)


POSITION_ENCODINGS.register("rope", RotaryEncoding)

__all__ = ["RotaryEncoding", "rope_inverse_frequencies"]
