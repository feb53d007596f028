"""How one request wants its tokens drawn.

The option names and their meanings are the reference's (kvcore/utils/sampling_params.py:8-26), so
a request written for it is accepted here unchanged.  What each option does in the batch sampler:

``max_tokens``   tokens to generate before the request ends with reason "length" (required, >= 1)
``temperature``  0 (anything below ``GREEDY_BELOW``) picks the largest logit; otherwise logits are
                 divided by it before the draw
``top_k``        keep the k largest logits (None: all)
``top_p``        keep the smallest set of most likely tokens whose probability reaches p
``seed``         makes the request's draws reproducible whatever else is in the batch
``skip_reading_prefix_cache``  never start this request from pages another request computed
``extra_args``   carried along untouched
"""
from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any, Mapping

GREEDY_BELOW = 1e-5   # the reference's threshold (kvcore/sample/sampler.py:11)

# option -> (test of a set value, what the message says it must be)
_RULES = {
    "max_tokens": (lambda v: v > 0, "positive"),
    "temperature": (lambda v: v >= 0, "non-negative"),
    "top_p": (lambda v: 0 < v <= 1, "in (0, 1]"),
    "top_k": (lambda v: v is None or v > 0, "positive when set"),
}


@dataclass(frozen=True, slots=True)
class SamplingParams:
    max_tokens: int
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int | None = None
    seed: int | None = None
    skip_reading_prefix_cache: bool | None = None
    extra_args: Mapping[str, Any] | None = None

    def __post_init__(self) -> None:
        for option, (accepts, wanted) in _RULES.items():
            value = getattr(self, option)
            if not accepts(value):
                raise ValueError(f"{option} must be {wanted}, got {value}")

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW

    def kept_logits(self, vocab_size: int) -> int:
        """Number of logits that survive ``top_k`` in a vocabulary of ``vocab_size``."""
        return vocab_size if self.top_k is None else min(self.top_k, vocab_size)

    @classmethod
    def from_mapping(cls, options: Mapping[str, Any]) -> "SamplingParams":
        """From a JSON-style mapping; an unknown option is an error that names it."""
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(options) - known)
        if unknown:
            raise ValueError(f"unknown sampling option(s): {', '.join(unknown)}; known: {', '.join(sorted(known))}")
        return cls(**dict(options))


__all__ = ["GREEDY_BELOW", "SamplingParams"]
