"""RMS normalisation with the residual sum folded in.

Formula as the reference computes it (kvcore/model/layer/rmsnorm.py:19-26): the optional
residual is added first and becomes the new residual; then in 32-bit
``y = x * rsqrt(mean(x^2) + eps)`` and ``out = (weight * y)`` cast to the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import NORMS, Norm, WeightSlot


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, *, size: int, eps: float, name: str, dtype: torch.dtype, device: torch.device):
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.weight = torch.empty(self.size, dtype=dtype, device=device)

    def _rebind(self, tensor: torch.Tensor) -> None:
        self.weight = tensor

    def weight_slots(self) -> list[WeightSlot]:
        return [
            WeightSlot(f"{self.name}.weight", self.weight, init="ones", keep_f32=True, rebind=self._rebind)
        ]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return K.rmsnorm(x, self.weight, self.eps)

    def forward_residual(self, h: torch.Tensor, residual: torch.Tensor):
        return K.add_rmsnorm(h, residual, self.weight, self.eps), residual

    def as_rms_scale(self):
        return self.weight, self.eps


NORMS.register("rmsnorm", RMSNorm)

__all__ = ["RMSNorm"]
