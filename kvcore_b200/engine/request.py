"""Scheduler-side state of one request.

The names the scheduler and its callers use are the reference's (kvcore/utils/request.py:13-46,
78-215): ``RequestStatus`` with its finished states, ``FinishReason``, and a ``Request`` that counts
its prompt, output and computed tokens.  A request here keeps one token list (prompt, then every
sampled token) and derives the rest from it; what the reference carries for streaming, priorities,
speculative tokens and transfers between engines has no user in this engine and is left out.
"""
from __future__ import annotations

import enum
import time
from typing import Sequence

from ..sampling.params import SamplingParams


class FinishReason(enum.StrEnum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    ERROR = "error"


class RequestStatus(enum.IntEnum):
    """Life of a request; every state after ``PREEMPTED`` is final and maps to a ``FinishReason``."""

    WAITING = 1
    RUNNING = 2
    PREEMPTED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH_CAPPED = 5
    FINISHED_ABORTED = 6
    FINISHED_ERROR = 7

    @staticmethod
    def is_finished(status: "RequestStatus") -> bool:
        return status >= RequestStatus.FINISHED_STOPPED

    @staticmethod
    def finish_reason(status: "RequestStatus") -> FinishReason | None:
        if not RequestStatus.is_finished(status):
            return None
        return (FinishReason.STOP, FinishReason.LENGTH, FinishReason.ABORT,
                FinishReason.ERROR)[status - RequestStatus.FINISHED_STOPPED]


class Request:
    """Tokens and progress of one request.

    ``num_computed_tokens`` is how many of ``all_token_ids`` have their keys and values in the cache;
    the request is in prefill while that is below ``num_prompt_tokens``."""

    def __init__(self, request_id: str, prompt_token_ids: Sequence[int], sampling_params: SamplingParams,
                 *, arrival_time: float | None = None) -> None:
        tokens = list(prompt_token_ids)
        if not tokens:
            raise ValueError("prompt_token_ids must be non-empty")
        self.request_id = request_id
        self.sampling_params = sampling_params
        self.arrival_time = arrival_time if arrival_time is not None else time.time()
        self.status = RequestStatus.WAITING
        self.num_prompt_tokens = len(tokens)
        self.num_computed_tokens = 0
        self.num_preemptions = 0
        self._tokens = tokens

    # ---- tokens ------------------------------------------------------------------------------
    @property
    def max_tokens(self) -> int:
        return self.sampling_params.max_tokens

    @property
    def all_token_ids(self) -> list[int]:
        """Prompt followed by the sampled tokens (the list itself, not a copy)."""
        return self._tokens

    @property
    def prompt_token_ids(self) -> list[int]:
        return self._tokens[: self.num_prompt_tokens]

    @property
    def output_token_ids(self) -> tuple[int, ...]:
        return tuple(self._tokens[self.num_prompt_tokens :])

    @property
    def num_tokens(self) -> int:
        return len(self._tokens)

    @property
    def num_output_tokens(self) -> int:
        return len(self._tokens) - self.num_prompt_tokens

    def append_output_token_id(self, token_id: int) -> None:
        self._tokens.append(token_id)

    # ---- ending ------------------------------------------------------------------------------
    def is_finished(self) -> bool:
        return RequestStatus.is_finished(self.status)

    def mark_finished(self, status: RequestStatus) -> None:
        if not RequestStatus.is_finished(status):
            raise ValueError(f"status must be a finished status, got {status}")
        self.status = status

    def get_finished_reason(self) -> FinishReason | None:
        return RequestStatus.finish_reason(self.status)


__all__ = ["FinishReason", "Request", "RequestStatus"]
