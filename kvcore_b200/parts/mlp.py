"""Gated feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up in one matrix.

The arithmetic is the reference's (kvcore/model/models/llama3.py:25-45;
kvcore/model/layer/activation.py:8-17).  The packing differs: when the intermediate size is a
multiple of 8, gate and up rows alternate in runs of 8 (gate 0-7, up 0-7, gate 8-15, ...), so that
the decode kernel, whose threads hold rows n and n+8 of a 16-row tile, can apply the activation
in its epilogue; otherwise rows ``[0, I)`` are the gate projection and ``[I, 2I)`` the up projection.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import FEED_FORWARDS, FeedForward, Summed, WeightSlot


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(
        self,
        *,
        hidden_size: int,
        intermediate_size: int,
        name: str,
        bias: bool = False,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.name = name
        inter = self.intermediate_size
        self.group = 8 if inter % 8 == 0 else 0      # run length of the gate/up interleave (0: halves)
        self.gate_up_weight = torch.empty(2 * inter, self.hidden_size, dtype=dtype, device=device)
        self.down_weight = torch.empty(self.hidden_size, inter, dtype=dtype, device=device)
        self.gate_up_bias = torch.empty(2 * inter, dtype=dtype, device=device) if bias else None
        self.down_bias = torch.empty(self.hidden_size, dtype=dtype, device=device) if bias else None

    def _halves(self, packed: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Where the gate and the up tensor go inside a packed ``[2I, ...]`` tensor."""
        inter, group = self.intermediate_size, self.group
        if group == 0:
            return packed[:inter], packed[inter:]
        runs = packed.view(inter // group, 2, group, *packed.shape[1:])
        return runs[:, 0], runs[:, 1]

    def weight_slots(self) -> list[WeightSlot]:
        inter, hidden = self.intermediate_size, self.hidden_size
        gate, up = self._halves(self.gate_up_weight)
        slots = [
            WeightSlot(f"{self.name}.gate_proj.weight", gate, file_shape=(inter, hidden)),
            WeightSlot(f"{self.name}.up_proj.weight", up, file_shape=(inter, hidden)),
            WeightSlot(f"{self.name}.down_proj.weight", self.down_weight),
        ]
        if self.gate_up_bias is not None:
            gate_bias, up_bias = self._halves(self.gate_up_bias)
            slots += [
                WeightSlot(f"{self.name}.gate_proj.bias", gate_bias, init="normal", file_shape=(inter,)),
                WeightSlot(f"{self.name}.up_proj.bias", up_bias, init="normal", file_shape=(inter,)),
                WeightSlot(f"{self.name}.down_proj.bias", self.down_bias, init="normal"),
            ]
        return slots

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        hidden = K.linear_silu_mul(x, self.gate_up_weight, self.gate_up_bias, group=self.group)
        return K.linear(hidden, self.down_weight, self.down_bias)


    def forward_prenorm(self, h, residual, rms_scale, ctx):
        """The layer's norm folded into the gate/up product and the residual sum into the down
        product (decode-sized batches: no kernel of their own for either)."""
        weight, eps = rms_scale
        summed = isinstance(h, Summed)
        hidden, residual = K.norm_linear(None if summed else h, residual, weight, eps, self.gate_up_weight,
                                         self.gate_up_bias, silu_group=self.group,
                                         sumsq=h.sumsq if summed else None)
        pending, sumsq = K.linear_add_residual(hidden, self.down_weight, self.down_bias, residual)
        return (Summed(sumsq) if pending is None else pending), residual


FEED_FORWARDS.register("swiglu", SwiGLU)

__all__ = ["SwiGLU"]
