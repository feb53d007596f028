"""Scheduler-side state of one request (reference: kvcore/utils/request.py:13-46, 78-215)."""
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
    WAITING = enum.auto()
    RUNNING = enum.auto()
    PREEMPTED = enum.auto()
    FINISHED_STOPPED = enum.auto()
    FINISHED_LENGTH_CAPPED = enum.auto()
    FINISHED_ABORTED = enum.auto()
    FINISHED_ERROR = enum.auto()

    @staticmethod
    def is_finished(status: "RequestStatus") -> bool:
        return status > RequestStatus.PREEMPTED

    @staticmethod
    def finish_reason(status: "RequestStatus") -> FinishReason | None:
        return _FINISH_REASONS.get(status)


_FINISH_REASONS = {
    RequestStatus.FINISHED_STOPPED: FinishReason.STOP,
    RequestStatus.FINISHED_LENGTH_CAPPED: FinishReason.LENGTH,
    RequestStatus.FINISHED_ABORTED: FinishReason.ABORT,
    RequestStatus.FINISHED_ERROR: FinishReason.ERROR,
}


class Request:
    def __init__(
        self,
        request_id: str,
        prompt_token_ids: Sequence[int],
        sampling_params: SamplingParams,
        *,
        arrival_time: float | None = None,
    ) -> None:
        if not prompt_token_ids:
            raise ValueError("prompt_token_ids must be non-empty")
        self.request_id = request_id
        self.sampling_params = sampling_params
        self.max_tokens = sampling_params.max_tokens
        self.arrival_time = time.time() if arrival_time is None else arrival_time
        self.status = RequestStatus.WAITING
        self.prompt_token_ids = list(prompt_token_ids)
        self.num_prompt_tokens = len(self.prompt_token_ids)
        self._output_token_ids: list[int] = []
        self._all_token_ids: list[int] = list(self.prompt_token_ids)
        self.num_computed_tokens = 0
        self.num_preemptions = 0

    @property
    def output_token_ids(self) -> tuple[int, ...]:
        return tuple(self._output_token_ids)

    @property
    def all_token_ids(self) -> list[int]:
        return self._all_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self._all_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self._output_token_ids)

    def append_output_token_id(self, token_id: int) -> None:
        self._output_token_ids.append(token_id)
        self._all_token_ids.append(token_id)

    def is_finished(self) -> bool:
        return RequestStatus.is_finished(self.status)

    def mark_finished(self, status: RequestStatus) -> None:
        if not RequestStatus.is_finished(status):
            raise ValueError(f"status must be a finished status, got {status}")
        self.status = status

    def get_finished_reason(self) -> FinishReason | None:
        return RequestStatus.finish_reason(self.status)


__all__ = ["FinishReason", "Request", "RequestStatus"]
