"""Gated feed-forward: ``down(silu(gate(x)) * up(x))`` with gate and up in one matrix.

As the reference (kvcore/model/models/llama3.py:25-45; kvcore/model/layer/activation.py:8-17):
rows ``[0, I)`` of the packed matrix are the gate projection, rows ``[I, 2I)`` the up projection.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import FEED_FORWARDS, FeedForward, WeightSlot


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
        self.gate_up_weight = torch.empty(2 * inter, self.hidden_size, dtype=dtype, device=device)
        self.down_weight = torch.empty(self.hidden_size, inter, dtype=dtype, device=device)
        self.gate_up_bias = torch.empty(2 * inter, dtype=dtype, device=device) if bias else None
        self.down_bias = torch.empty(self.hidden_size, dtype=dtype, device=device) if bias else None

    def weight_slots(self) -> list[WeightSlot]:
        inter = self.intermediate_size
        slots = [
            WeightSlot(f"{self.name}.gate_proj.weight", self.gate_up_weight[:inter]),
            WeightSlot(f"{self.name}.up_proj.weight", self.gate_up_weight[inter:]),
            WeightSlot(f"{self.name}.down_proj.weight", self.down_weight),
        ]
        if self.gate_up_bias is not None:
            slots += [
                WeightSlot(f"{self.name}.gate_proj.bias", self.gate_up_bias[:inter], init="normal"),
                WeightSlot(f"{self.name}.up_proj.bias", self.gate_up_bias[inter:], init="normal"),
                WeightSlot(f"{self.name}.down_proj.bias", self.down_bias, init="normal"),
            ]
        return slots

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        gate_up = K.linear(x, self.gate_up_weight, self.gate_up_bias)
        return K.linear(K.silu_mul(gate_up), self.down_weight, self.down_bias)


FEED_FORWARDS.register("swiglu", SwiGLU)

__all__ = ["SwiGLU"]
