"""The decoder assembled from a ``ModelSpec``: embedding, blocks run in schedule order,
final norm and output head.

Flow as the reference's model (kvcore/model/models/llama3.py:182-200, 245-247): embed, run
the blocks carrying ``(h, residual)``, and fold the last residual into the final norm.
Here only the rows whose logits are wanted go through the final norm and the head.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..config.model_spec import ModelSpec
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the stock parts)
from .base import BLOCKS, EMBEDDINGS, LM_HEADS, NORMS, CacheSpec, StateSpec, Summed, WeightSlot


@dataclass(frozen=True)
class EntryRequirement:
    """What one schedule entry needs cached: paged keys/values, fixed-size state, or a borrowed cache."""

    entry: int
    layer: int
    cache_spec: CacheSpec | None
    state_spec: StateSpec | None
    cache_of: int | None


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device: torch.device) -> None:
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.embedding = EMBEDDINGS.build(spec.embedding, dtype=dtype, device=device)
        self.blocks = [
            BLOCKS.build(layer.block, layer=layer, dtype=dtype, device=device) for layer in spec.layers
        ]
        self.final_norm = NORMS.build(spec.final_norm, dtype=dtype, device=device)
        tied_to = spec.lm_head.params.get("tied_to")
        tied_weight = None
        if tied_to is not None:
            if tied_to != spec.embedding.params.get("name"):
                raise ValueError(f"lm head is tied to {tied_to!r}, which is not the embedding")
            tied_weight = self.embedding.weight
        self.lm_head = LM_HEADS.build(spec.lm_head, tied_weight=tied_weight, dtype=dtype, device=device)
        self.schedule = spec.schedule

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph."""
        return all(part.graph_safe for part in self._parts())

    # ---- weights -------------------------------------------------------------------------
    def _parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.lm_head]

    def weight_slots(self) -> list[WeightSlot]:
        slots: list[WeightSlot] = []
        for part in self._parts():
            slots += part.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        names: list[str] = []
        for part in self._parts():
            names += part.ignorable_tensor_names()
        return names

    def finalize_weights(self) -> None:
        for part in self._parts():
            part.finalize_weights()

    def state_dict(self) -> dict[str, torch.Tensor]:
        """The model's tensors under their checkpoint names and in their checkpoint shapes, on the
        model's device (packed matrices are split and scattered rows gathered again; copies where a
        slot is a strided view)."""
        return {slot.name: slot.dest.reshape(slot.shape) for slot in self.weight_slots()}

    def weight_bytes(self) -> int:
        seen: set[int] = set()
        total = 0
        for slot in self.weight_slots():
            base = slot.dest.untyped_storage().data_ptr() if slot.dest.device.type != "meta" else id(slot)
            if (base, slot.dest.storage_offset()) in seen:
                continue
            seen.add((base, slot.dest.storage_offset()))
            total += slot.dest.numel() * slot.dest.element_size()
        return total

    # ---- cache needs -----------------------------------------------------------------------
    def entry_requirements(self) -> list[EntryRequirement]:
        out = []
        for index, entry in enumerate(self.schedule):
            mixer = self.blocks[entry.layer].mixer
            out.append(
                EntryRequirement(index, entry.layer, mixer.cache_spec(), mixer.state_spec(), entry.cache_of)
            )
        return out

    # ---- the forward pass of one step --------------------------------------------------------
    def forward(self, ctx, caches) -> tuple[torch.Tensor, torch.Tensor]:
        """Run the step's tokens through every schedule entry; returns ``(h, residual)``."""
        h = self.embedding.forward(ctx.token_ids)
        residual = None
        for index, entry in enumerate(self.schedule):
            h, residual = self.blocks[entry.layer].forward(h, residual, ctx, caches[index])
        return h, residual

    def compute_logits(self, h: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[len(rows), V]`` of the token rows ``rows`` (int32 indices)."""
        residual_rows = K.gather_rows(residual, rows)
        if isinstance(h, Summed):      # the last sub-layer has added its output into the residual itself
            normed = self.final_norm.forward(residual_rows)
        else:
            normed, _ = self.final_norm.forward_residual(K.gather_rows(h, rows), residual_rows)
        return self.lm_head.forward(normed)


def build_model(spec: ModelSpec, *, dtype: torch.dtype, device: torch.device | str) -> DecoderModel:
    return DecoderModel(spec, dtype=dtype, device=torch.device(device))


__all__ = ["DecoderModel", "EntryRequirement", "build_model"]
