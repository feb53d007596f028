"""One engine step: schedule, run the model, sample, update request state.

Same loop as the reference's engine core (kvcore/engine/engine_core.py:38-152, 209-217): the
scheduler owns request state and the cache manager's bookkeeping, the runner owns the model
and the cache tensors; stop tokens come from config.json's ``eos_token_id`` and from the
tokenizer when there is one.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

from ..config.engine_config import KVCoreConfig
from ..sampling.params import SamplingParams
from ..utils.tokenizer import TokenizerManager
from .request import FinishReason, Request
from .runner import ModelRunner
from .scheduler import RequestStepOutput, Scheduler

logger = logging.getLogger("kvcore_b200.engine")


@dataclass(frozen=True)
class EngineCoreOutputs:
    request_outputs: tuple[RequestStepOutput, ...] = ()


@dataclass(frozen=True)
class FinishedRequestOutput:
    request_id: str
    output_token_ids: tuple[int, ...]
    finish_reason: FinishReason | None


class EngineCore:
    def __init__(self, config: KVCoreConfig, *, model_runner: ModelRunner | None = None) -> None:
        self.config = config
        self.model_runner = model_runner if model_runner is not None else ModelRunner(config)
        self.tokenizer_manager = TokenizerManager(config.model_config.model)
        self.stop_token_ids = set(self.tokenizer_manager.get_stop_token_ids())
        self.stop_token_ids.update(self.model_runner.model.spec.eos_token_ids)
        self.scheduler = Scheduler(config.scheduler_config, self.model_runner.kv_manager)
        self.finished_outputs: dict[str, FinishedRequestOutput] = {}

    def add_request(
        self,
        request_id: str,
        sampling_params: SamplingParams,
        *,
        prompt_token_ids: Sequence[int] | None = None,
        messages: Sequence[Mapping[str, Any]] | None = None,
    ) -> None:
        if prompt_token_ids is None:
            if messages is None:
                raise ValueError("a request needs prompt_token_ids or messages")
            prompt_token_ids = self.tokenizer_manager.encode_messages(messages)
        vocab = self.model_runner.model.spec.vocab_size
        for token in prompt_token_ids:
            if not 0 <= int(token) < vocab:
                raise ValueError(f"request {request_id!r}: token id {token} is outside [0, {vocab})")
        self.scheduler.add_request(Request(request_id, [int(t) for t in prompt_token_ids], sampling_params))

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    def step(self) -> EngineCoreOutputs:
        scheduler_output = self.scheduler.schedule()
        if scheduler_output.total_num_scheduled_tokens == 0:
            self.model_runner.remove_requests(scheduler_output.finished_req_ids)
            self.model_runner.remove_requests(scheduler_output.preempted_req_ids)
            return EngineCoreOutputs()
        self.model_runner.execute_model(scheduler_output)
        runner_output = self.model_runner.sample_tokens()
        sampled = {
            req_id: tokens[0]
            for req_id, tokens in zip(runner_output.req_ids, runner_output.sampled_token_ids)
            if tokens
        }
        update = self.scheduler.update_from_outputs(
            scheduler_output, sampled, stop_token_ids=self.stop_token_ids
        )
        for finished in update.finished_requests:
            self.finished_outputs[finished.request_id] = FinishedRequestOutput(
                finished.request_id, finished.output_token_ids, finished.finish_reason
            )
        self.model_runner.remove_requests([f.request_id for f in update.finished_requests])
        return EngineCoreOutputs(update.step_outputs)

    def take_finished_output(self, request_id: str) -> FinishedRequestOutput | None:
        return self.finished_outputs.pop(request_id, None)


__all__ = ["EngineCore", "EngineCoreOutputs", "FinishedRequestOutput"]
