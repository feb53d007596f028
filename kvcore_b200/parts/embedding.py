"""Token embedding and output head.

Embedding is a row gather (kvcore/model/models/llama3.py:161-165, 178-180).  The head
multiplies the selected hidden rows with the ``[V, E]`` matrix, shares the embedding matrix
when tied, and applies ``logit_scale`` when it is not 1 (llama3.py:219-225, 245-247;
kvcore/sample/logits_processor.py:46-54).  Logits leave the head in 32-bit.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import EMBEDDINGS, LM_HEADS, Part, WeightSlot


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, name: str, dtype, device) -> None:
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        self.weight = torch.empty(self.vocab_size, self.hidden_size, dtype=dtype, device=device)

    def weight_slots(self) -> list[WeightSlot]:
        return [WeightSlot(f"{self.name}.weight", self.weight)]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return K.gather_rows(self.weight, token_ids)


class LMHead(Part):
    graph_safe = True

    def __init__(
        self,
        *,
        vocab_size: int,
        hidden_size: int,
        name: str,
        tied_to: str | None = None,
        logit_scale: float = 1.0,
        tied_weight: torch.Tensor | None = None,
        dtype,
        device,
    ) -> None:
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        self.tied_to = tied_to
        self.logit_scale = float(logit_scale)
        if tied_to is not None:
            if tied_weight is None:
                raise ValueError(f"lm head is tied to {tied_to!r} but no such matrix was given")
            self.weight = tied_weight
        else:
            self.weight = torch.empty(self.vocab_size, self.hidden_size, dtype=dtype, device=device)

    def weight_slots(self) -> list[WeightSlot]:
        if self.tied_to is not None:
            return []
        return [WeightSlot(f"{self.name}.weight", self.weight)]

    def ignorable_tensor_names(self) -> list[str]:
        # a checkpoint may still carry the tied matrix under the head's own name
        return [f"{self.name}.weight"] if self.tied_to is not None else []

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        logits = K.linear(hidden, self.weight, None, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            logits = logits * self.logit_scale
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
LM_HEADS.register("lm_head", LMHead)

__all__ = ["LMHead", "TokenEmbedding"]
