"""Next-token sampling from 32-bit logits: greedy, temperature, top-k, top-p, seeded.

Rule as the reference's sampler (kvcore/sample/sampler.py:86-167): a temperature below
1e-5 means greedy argmax; otherwise logits are divided by the temperature, all but the k
largest are masked (top-k), then the smallest-probability tokens whose cumulative
probability stays <= 1 - p are masked (top-p, the largest always kept), and the token is
``argmax(softmax(logits) / q)`` with ``q ~ Exp(1)`` per vocabulary entry.

Deliberate difference: the reference rebuilds a seeded generator at every call, so a
seeded request sees the same noise at every decode step (sampler.py:53-57, 185-188).  Here
the noise is a counter-based stream keyed by (request seed, index of the token being
sampled, vocabulary entry), so a seeded request is reproducible and does not depend on
what else is in the batch.  One kernel launch samples the whole batch.
"""
from __future__ import annotations

import random
from typing import Sequence

import torch

from .. import kernels as K
from .params import GREEDY_BELOW, SamplingParams

SAMPLING_EPS = GREEDY_BELOW  # one threshold for the host's view and the kernel's


class Sampler:
    def __init__(self, device: torch.device | str) -> None:
        self.device = torch.device(device)
        # On a CUDA device the rows' parameters travel through two pinned buffers in turn, copied
        # without waiting, so that a caller who does not read the tokens back (a pipelined loop)
        # is never held up by the device.
        self._staging: list[torch.Tensor] = []
        self._on_device: list[torch.Tensor] = []
        self._copied: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0

    def _upload(self, packed: torch.Tensor) -> torch.Tensor:
        """``packed [rows, 6]`` float64 on the host -> the same on the device, asynchronously."""
        if self.device.type != "cuda":
            return packed
        rows = packed.shape[0]
        if not self._staging or self._staging[0].shape[0] < rows:
            capacity = max(64, rows)
            self._staging = [torch.empty((capacity, 6), dtype=torch.float64, pin_memory=True) for _ in range(2)]
            self._on_device = [torch.empty((capacity, 6), dtype=torch.float64, device=self.device) for _ in range(2)]
            self._copied = [None, None]
        turn = self._turn
        self._turn ^= 1
        if self._copied[turn] is not None:
            self._copied[turn].synchronize()           # the copy that last used this buffer has run
        self._staging[turn][:rows].copy_(packed)
        target = self._on_device[turn][:rows]
        target.copy_(self._staging[turn][:rows], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._copied[turn] = event
        return target

    @staticmethod
    def fresh_seed() -> int:
        """A seed for a request that gave none."""
        return random.getrandbits(62)

    def sample(
        self,
        logits: torch.Tensor,
        params: Sequence[SamplingParams],
        seeds: Sequence[int],
        token_indices: Sequence[int],
    ) -> torch.Tensor:
        """``logits [S, V]`` 32-bit -> int32 ``[S]`` token ids.

        ``seeds[i]`` and ``token_indices[i]`` (how many tokens request i has sampled so far)
        select the noise stream of row i.
        """
        if logits.dim() != 2:
            raise ValueError(f"logits must be [rows, vocab], got {tuple(logits.shape)}")
        rows, vocab = logits.shape
        if not (len(params) == len(seeds) == len(token_indices) == rows):
            raise ValueError("one SamplingParams, seed and token index per logits row is needed")
        if logits.dtype != torch.float32:
            logits = logits.float()
        packed = torch.tensor(
            [
                (
                    p.temperature,
                    p.kept_logits(vocab),
                    p.top_p,
                    float(int(seed) & 0xFFFFFFFF),
                    float((int(seed) >> 32) & 0xFFFFFFFF),
                    index,
                )
                for p, seed, index in zip(params, seeds, token_indices)
            ],
            dtype=torch.float64,
        )
        return K.sample(logits, self._upload(packed), SAMPLING_EPS)


__all__ = ["SAMPLING_EPS", "Sampler"]
