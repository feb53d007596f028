"""Grouped-query attention over the paged cache.

Order of operations as in the reference's attention layer
(kvcore/model/models/llama3.py:87-104; kvcore/model/layer/attention.py:53-96;
kvcore/model/attn_backend/torch_paged.py:90-117, 151-166): one packed q/k/v projection,
position encoding on q and k, keys and values of this step's tokens written into their
pages, then every query attends over its request's cached positions up to its own
(optionally only the trailing ``sliding_window`` of them) with 32-bit scores, softmax and
accumulation, and the output projection.  Query head ``h`` reads kv head ``h // (H/KVH)``.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from ..config.model_spec import PartSpec
from .base import MIXERS, POSITION_ENCODINGS, CacheSpec, Mixer, Summed, WeightSlot


class PagedAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    def __init__(
        self,
        *,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        name: str,
        bias: bool = False,
        sliding_window: int | None = None,
        position: PartSpec | None = None,
        dtype: torch.dtype,
        device: torch.device,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} must be a multiple of num_kv_heads {num_kv_heads}")
        if sliding_window is not None and sliding_window <= 0:
            raise ValueError(f"sliding_window must be positive when set, got {sliding_window}")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.sliding_window = None if sliding_window is None else int(sliding_window)
        self.name = name
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        K.check_attention_shape(self.num_heads, self.num_kv_heads, self.head_dim, dtype)
        self.qkv_weight = torch.empty(
            self.q_size + 2 * self.kv_size, self.hidden_size, dtype=dtype, device=device
        )
        self.o_weight = torch.empty(self.hidden_size, self.q_size, dtype=dtype, device=device)
        self.qkv_bias = (
            torch.empty(self.q_size + 2 * self.kv_size, dtype=dtype, device=device) if bias else None
        )
        self.o_bias = torch.empty(self.hidden_size, dtype=dtype, device=device) if bias else None
        self.position = (
            None
            if position is None
            else POSITION_ENCODINGS.build(position, dtype=dtype, device=device)
        )

    def cache_spec(self) -> CacheSpec:
        return CacheSpec.keys_and_values(self.num_kv_heads, self.head_dim, self.sliding_window)

    def weight_slots(self) -> list[WeightSlot]:
        q, kv = self.q_size, self.kv_size
        slots = [
            WeightSlot(f"{self.name}.q_proj.weight", self.qkv_weight[:q]),
            WeightSlot(f"{self.name}.k_proj.weight", self.qkv_weight[q : q + kv]),
            WeightSlot(f"{self.name}.v_proj.weight", self.qkv_weight[q + kv :]),
            WeightSlot(f"{self.name}.o_proj.weight", self.o_weight),
        ]
        if self.qkv_bias is not None:
            slots += [
                WeightSlot(f"{self.name}.q_proj.bias", self.qkv_bias[:q], init="normal"),
                WeightSlot(f"{self.name}.k_proj.bias", self.qkv_bias[q : q + kv], init="normal"),
                WeightSlot(f"{self.name}.v_proj.bias", self.qkv_bias[q + kv :], init="normal"),
                WeightSlot(f"{self.name}.o_proj.bias", self.o_bias, init="normal"),
            ]
        if self.position is not None:
            slots += self.position.weight_slots()
        return slots

    def ignorable_tensor_names(self) -> list[str]:
        return [] if self.position is None else self.position.ignorable_tensor_names()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        out = self._attend(K.linear(x, self.qkv_weight, self.qkv_bias), ctx, cache)
        return K.linear(out, self.o_weight, self.o_bias)

    def forward_prenorm(self, h, residual, rms_scale, ctx, cache):
        """The layer's norm folded into the q/k/v product and the residual sum into the output
        product (decode-sized batches: no kernel of their own for either)."""
        weight, eps = rms_scale
        summed = isinstance(h, Summed)
        qkv, residual = K.norm_linear(None if summed else h, residual, weight, eps, self.qkv_weight, self.qkv_bias,
                                      sumsq=h.sumsq if summed else None)
        out = self._attend(qkv, ctx, cache)
        pending, sumsq = K.linear_add_residual(out, self.o_weight, self.o_bias, residual)
        return (Summed(sumsq) if pending is None else pending), residual

    def _attend(self, qkv: torch.Tensor, ctx, cache) -> torch.Tensor:
        table = ctx.block_table(cache.group)
        # an encoding that offers its angles as a table gets its rotation fused with the cache write
        cos_sin = None if self.position is None else self.position.cos_sin(ctx)
        if cos_sin is None and self.position is not None:
            tokens = qkv.shape[0]
            q = qkv[:, : self.q_size].view(tokens, self.num_heads, self.head_dim)
            k = qkv[:, self.q_size : self.q_size + self.kv_size].view(
                tokens, self.num_kv_heads, self.head_dim
            )
            self.position.apply(q, k if cache.owner else None, ctx)
        # rotation and cache write run inside the decode kernel where that one is taken, in a
        # kernel in front of the attention otherwise
        return K.paged_attention(
            qkv, cache.k, cache.v, table, ctx,
            self.num_heads, self.num_kv_heads, self.head_dim, self.scale, self.sliding_window,
            cos_sin=cos_sin, write_kv=cache.owner,
        )


MIXERS.register("paged_attention", PagedAttention)

__all__ = ["PagedAttention"]
