"""Arrangement of one layer: pre-norm mixer and feed-forward on a deferred residual.

As the reference's decoder layer (kvcore/model/models/llama3.py:124-142): the running
``residual`` and the last sub-layer output ``h`` stay separate and are summed inside the
next norm; the first block starts with ``residual = h``.
"""
from __future__ import annotations

import torch

from ..config.model_spec import LayerSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Summed, WeightSlot


class PreNormResidualBlock(Block):
    def __init__(self, *, layer: LayerSpec, dtype: torch.dtype, device: torch.device) -> None:
        self.mixer_norm = NORMS.build(layer.norms["mixer_norm"], dtype=dtype, device=device)
        self.mixer = MIXERS.build(layer.mixer, dtype=dtype, device=device)
        self.feed_forward_norm = NORMS.build(layer.norms["feed_forward_norm"], dtype=dtype, device=device)
        self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, dtype=dtype, device=device)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def weight_slots(self) -> list[WeightSlot]:
        slots: list[WeightSlot] = []
        for part in self.parts():
            slots += part.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        names: list[str] = []
        for part in self.parts():
            names += part.ignorable_tensor_names()
        return names

    def finalize_weights(self) -> None:
        for part in self.parts():
            part.finalize_weights()

    def forward(self, h, residual, ctx, cache):
        # A part that can take its input before the norm (and fold the norm into its first matrix
        # product, the residual sum into its last) gets it that way; otherwise the norm runs as a
        # step of its own.  ``h`` may be ``Summed``: the part in front added its output already.
        scale, prenorm = self.mixer_norm.as_rms_scale(), getattr(self.mixer, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            a, residual = prenorm(h, residual, scale, ctx, cache)
        else:
            if isinstance(h, Summed):
                x = self.mixer_norm.forward(residual)
            elif residual is None:
                residual = h
                x = self.mixer_norm.forward(h)
            else:
                x, residual = self.mixer_norm.forward_residual(h, residual)
            a = self.mixer.forward(x, ctx, cache)
        scale, prenorm = self.feed_forward_norm.as_rms_scale(), getattr(self.feed_forward, "forward_prenorm", None)
        if scale is not None and prenorm is not None:
            h, residual = prenorm(a, residual, scale, ctx)
        else:
            if isinstance(a, Summed):
                x = self.feed_forward_norm.forward(residual)
            else:
                x, residual = self.feed_forward_norm.forward_residual(a, residual)
            h = self.feed_forward.forward(x, ctx)
        return h, residual


BLOCKS.register("prenorm_residual", PreNormResidualBlock)

__all__ = ["PreNormResidualBlock"]
