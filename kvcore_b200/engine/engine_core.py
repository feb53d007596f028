"""One engine step: schedule, run the model, sample, update request state.

Same loop as the reference's engine core (kvcore/engine/engine_core.py:38-152, 209-217): the
scheduler owns request state and the cache manager's bookkeeping, the runner owns the model
and the cache tensors; stop tokens come from config.json's ``eos_token_id`` and from the
tokenizer when there is one.

Not in the reference: with ``SchedulerConfig.run_ahead`` the core keeps one step in flight.  While
the device runs step k, the host plans step k+1 where that is possible without k's tokens
(``Scheduler.schedule_ahead``: a batch in steady decoding), launches it with the token ids fed
from the sampler's output on the device, and only then waits for k's tokens.  The device no
longer idles through the host's share of a step; ``step()`` still returns one step's outputs per
call, in order.  A request that stops on a token is seen one step late: the extra token it
computed meanwhile is dropped, so outputs are the same as without running ahead.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

from ..config.engine_config import KVCoreConfig
from ..sampling.params import SamplingParams
from ..utils.tokenizer import TokenizerManager
from .request import FinishReason, Request, RequestStatus
from .runner import ModelRunner, SampleHandle
from .scheduler import RequestStepOutput, Scheduler, SchedulerOutput

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
        self.run_ahead = bool(config.scheduler_config.run_ahead)
        self._in_flight: tuple[SchedulerOutput, SampleHandle] | None = None
        self.num_steps_run_ahead = 0

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

    def _launch(self, plan: SchedulerOutput, feed: SampleHandle | None = None) -> tuple[SchedulerOutput, SampleHandle]:
        self.model_runner.execute_model(plan, feed)
        return plan, self.model_runner.launch_sampling()

    def step(self) -> EngineCoreOutputs:
        if self._in_flight is None:
            plan = self.scheduler.schedule()
            if plan.total_num_scheduled_tokens == 0:
                self.model_runner.remove_requests(plan.finished_req_ids)
                self.model_runner.remove_requests(plan.preempted_req_ids)
                return EngineCoreOutputs()
            self._in_flight = self._launch(plan)
        plan, handle = self._in_flight
        ahead = None
        if self.run_ahead:
            next_plan = self.scheduler.schedule_ahead(plan)
            if next_plan is not None:
                ahead = self._launch(next_plan, feed=handle)
                self.num_steps_run_ahead += 1
        runner_output = self.model_runner.collect(handle)
        sampled = {
            req_id: tokens[0]
            for req_id, tokens in zip(runner_output.req_ids, runner_output.sampled_token_ids)
            if tokens
        }
        update = self.scheduler.update_from_outputs(plan, sampled, stop_token_ids=self.stop_token_ids)
        for finished in update.finished_requests:
            self.finished_outputs[finished.request_id] = FinishedRequestOutput(
                finished.request_id, finished.output_token_ids, finished.finish_reason
            )
        self.model_runner.remove_requests([f.request_id for f in update.finished_requests])
        if ahead is not None and not any(r in self.scheduler.requests for r in ahead[0].num_scheduled_tokens):
            # every request of the step launched ahead has just ended: its tokens are nobody's
            self.model_runner.collect(ahead[1])
            self.model_runner.remove_requests(ahead[0].num_scheduled_tokens)
            ahead = None
        self._in_flight = ahead
        return EngineCoreOutputs(update.step_outputs)

    def drain(self) -> None:
        """Wait for a step that is still in flight and take its tokens in, so that nothing is pending."""
        if self._in_flight is None:
            return
        plan, handle = self._in_flight
        self._in_flight = None
        runner_output = self.model_runner.collect(handle)
        sampled = {r: t[0] for r, t in zip(runner_output.req_ids, runner_output.sampled_token_ids) if t}
        update = self.scheduler.update_from_outputs(plan, sampled, stop_token_ids=self.stop_token_ids)
        for finished in update.finished_requests:
            self.finished_outputs[finished.request_id] = FinishedRequestOutput(
                finished.request_id, finished.output_token_ids, finished.finish_reason
            )
        self.model_runner.remove_requests([f.request_id for f in update.finished_requests])

    def abort_requests(self, request_ids: Sequence[str] | None = None) -> tuple[FinishedRequestOutput, ...]:
        """End the given requests (all of them for ``None``) with reason "abort": their pages go back,
        what they generated so far is kept as their finished output.  A step in flight is taken in
        first, so a request may turn out to have ended by itself meanwhile."""
        self.drain()
        aborted = self.scheduler.finish_requests(
            None if request_ids is None else list(request_ids), RequestStatus.FINISHED_ABORTED
        )
        outputs = tuple(FinishedRequestOutput(f.request_id, f.output_token_ids, f.finish_reason) for f in aborted)
        for output in outputs:
            self.finished_outputs[output.request_id] = output
        self.model_runner.remove_requests([o.request_id for o in outputs])
        return outputs

    def take_finished_output(self, request_id: str) -> FinishedRequestOutput | None:
        return self.finished_outputs.pop(request_id, None)


__all__ = ["EngineCore", "EngineCoreOutputs", "FinishedRequestOutput"]
