"""Continuous-batching scheduler with chunked prefill under a token budget.

Policy and contract follow the reference (kvcore/sched/scheduler.py:147-302, 333-416,
418-577; kvcore/sched/utils.py:11-96): each ``schedule()`` first serves running requests in
order (one token for a decoding request, a portion of the prompt otherwise), then admits
waiting requests first-come-first-served, all under ``max_num_scheduled_tokens`` and
``max_num_seqs``; at most ``max_num_partial_prefills`` requests may be in prefill in one
step.  A request is new to the runner the step it leaves the waiting queue
(``NewRequestData``) and cached afterwards (``CachedRequestData``).

When pages run out (decided here, tested in tests/test_scheduler.py): a request that cannot
get pages is not scheduled this step, and, as in the reference, running requests behind it
wait too.  If nothing at all could be scheduled while requests are unfinished, the reference
only reports no progress (scheduler.py:263-273).  Here, with ``preempt_on_deadlock``, the
youngest running request is preempted instead: its pages are freed and it returns to the
front of the waiting queue to be recomputed from its tokens so far; the step is then
planned again.  A lone request that cannot fit even with every page free is a hard error.
Block ids are not part of the output: block tables are persistent rows of the shared cache
manager.
"""
from __future__ import annotations

import logging
from collections import deque
from dataclasses import dataclass, field
from typing import Iterable, Mapping

from ..cache.kv_manager import KVManager
from ..config.engine_config import SchedulerConfig
from ..sampling.params import SamplingParams
from .request import FinishReason, Request, RequestStatus

logger = logging.getLogger("kvcore_b200.scheduler")


@dataclass(frozen=True)
class NewRequestData:
    req_id: str
    prompt_token_ids: tuple[int, ...]
    sampling_params: SamplingParams
    num_computed_tokens: int
    num_output_tokens: int = 0


@dataclass(frozen=True)
class CachedRequestData:
    req_ids: tuple[str, ...] = ()
    new_token_ids: tuple[tuple[int, ...], ...] = ()
    num_computed_tokens: tuple[int, ...] = ()
    num_output_tokens: tuple[int, ...] = ()

    @property
    def num_reqs(self) -> int:
        return len(self.req_ids)


@dataclass(frozen=True)
class SchedulerOutput:
    scheduled_new_reqs: tuple[NewRequestData, ...] = ()
    scheduled_cached_reqs: CachedRequestData = field(default_factory=CachedRequestData)
    num_scheduled_tokens: dict[str, int] = field(default_factory=dict)
    total_num_scheduled_tokens: int = 0
    finished_req_ids: frozenset[str] = frozenset()
    preempted_req_ids: tuple[str, ...] = ()
    step_id: int = 0
    # requests whose one scheduled token is the one the step in front samples (plan made ahead)
    pending_token_req_ids: frozenset[str] = frozenset()

    @property
    def is_empty(self) -> bool:
        return self.total_num_scheduled_tokens == 0 and not self.finished_req_ids


@dataclass(frozen=True)
class RequestStepOutput:
    request_id: str
    sampled_token_id: int | None
    finished: bool
    finish_reason: FinishReason | None


@dataclass(frozen=True)
class FinishedRequestState:
    request_id: str
    output_token_ids: tuple[int, ...]
    finish_reason: FinishReason | None


@dataclass(frozen=True)
class SchedulerUpdateResult:
    step_outputs: tuple[RequestStepOutput, ...]
    finished_requests: tuple[FinishedRequestState, ...]


@dataclass(frozen=True)
class SchedulerNoProgressState:
    waiting: tuple[str, ...]
    running: tuple[str, ...]
    free_pages: tuple[int, ...]

    def format_message(self) -> str:
        return (
            f"Scheduler made no progress (waiting={self.waiting}, running={self.running}, "
            f"free_pages={self.free_pages})"
        )


class Scheduler:
    def __init__(self, config: SchedulerConfig, kv_manager: KVManager) -> None:
        self.config = config
        self.kv_manager = kv_manager
        self.requests: dict[str, Request] = {}
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished_req_ids: set[str] = set()
        self.last_no_progress_state: SchedulerNoProgressState | None = None
        self.step_id = 0
        self.num_preemptions = 0

    # ---- admission -----------------------------------------------------------------------------
    def add_request(self, request: Request) -> None:
        if request.request_id in self.requests:
            raise ValueError(f"Duplicate request_id: {request.request_id}")
        kv = self.kv_manager
        if request.num_prompt_tokens >= kv.max_model_len:
            raise ValueError(
                f"request {request.request_id!r}: prompt of {request.num_prompt_tokens} tokens leaves "
                f"no room to generate within max_model_len {kv.max_model_len}"
            )
        pages = -(-(request.num_prompt_tokens + 1) // kv.page_size)
        for group, pool in zip(kv.groups, kv.pools):
            if group.window is None and pages > pool.num_usable:
                raise ValueError(
                    f"request {request.request_id!r} needs {pages} pages for its prompt but the "
                    f"cache holds {pool.num_usable}: it can never be scheduled"
                )
        self.requests[request.request_id] = request
        self.waiting.append(request)

    def has_unfinished_requests(self) -> bool:
        return bool(self.running) or bool(self.waiting)

    def get_num_unfinished_requests(self) -> int:
        return len(self.running) + len(self.waiting)

    def get_request_counts(self) -> tuple[int, int]:
        return len(self.running), len(self.waiting)

    # ---- finishing -----------------------------------------------------------------------------
    def finish_requests(
        self, request_ids: str | Iterable[str] | None, finished_status: RequestStatus
    ) -> tuple[FinishedRequestState, ...]:
        if not RequestStatus.is_finished(finished_status):
            raise ValueError(f"finished_status must be a finished status, got {finished_status}")
        if isinstance(request_ids, str):
            ids = {request_ids}
        elif request_ids is None:
            ids = set(self.requests)
        else:
            ids = set(request_ids)
        finished = []
        for request_id in ids:
            request = self.requests.get(request_id)
            if request is None or request.is_finished():
                continue
            request.mark_finished(finished_status)
            finished.append(self._free_finished_request(request))
        return tuple(finished)

    def shutdown(self) -> None:
        self.finish_requests(None, RequestStatus.FINISHED_ABORTED)

    def _free_finished_request(self, request: Request) -> FinishedRequestState:
        self.kv_manager.free(request.request_id)
        self.running = [r for r in self.running if r.request_id != request.request_id]
        if request in self.waiting:
            self.waiting.remove(request)
        self.requests.pop(request.request_id, None)
        self.finished_req_ids.add(request.request_id)
        return FinishedRequestState(
            request_id=request.request_id,
            output_token_ids=request.output_token_ids,
            finish_reason=request.get_finished_reason(),
        )

    # ---- planning a step -------------------------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        self.last_no_progress_state = None
        preempted: list[str] = []
        while True:
            output = self._plan(preempted)
            if output is not None:
                return output
            # nothing could be scheduled and nothing finished
            victim = self._pick_preemption_victim()
            if victim is None:
                self.last_no_progress_state = SchedulerNoProgressState(
                    waiting=tuple(r.request_id for r in self.waiting),
                    running=tuple(r.request_id for r in self.running),
                    free_pages=tuple(self.kv_manager.num_free_pages()),
                )
                logger.warning(self.last_no_progress_state.format_message())
                return SchedulerOutput(preempted_req_ids=tuple(preempted), step_id=self.step_id)
            self._preempt(victim)
            preempted.append(victim.request_id)

    def _pick_preemption_victim(self) -> Request | None:
        if not self.config.preempt_on_deadlock or len(self.running) < 2:
            return None
        return self.running[-1]

    def _preempt(self, request: Request) -> None:
        logger.info("preempting request %s to free pages", request.request_id)
        self.kv_manager.free(request.request_id)
        self.running.remove(request)
        request.status = RequestStatus.PREEMPTED
        request.num_computed_tokens = 0
        request.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(request)

    def _plan(self, preempted: list[str]) -> SchedulerOutput | None:
        cfg = self.config
        token_budget = cfg.max_num_scheduled_tokens
        new_reqs: list[NewRequestData] = []
        cached_ids: list[str] = []
        cached_tokens: list[tuple[int, ...]] = []
        cached_computed: list[int] = []
        cached_outputs: list[int] = []
        num_scheduled: dict[str, int] = {}
        partial = 0
        long_partial = 0

        def try_schedule(request: Request, from_waiting: bool) -> tuple[int, bool] | None:
            nonlocal token_budget
            if token_budget <= 0:
                return None
            is_prefill = self._is_prefill(request)
            if is_prefill and not self._can_schedule_partial_prefill(request, partial, long_partial):
                return None
            # a request that starts (or starts again): pages that already hold its first tokens
            prefix_pages: list[tuple[int, ...]] = []
            if (from_waiting and request.num_computed_tokens == 0
                    and not request.sampling_params.skip_reading_prefix_cache):
                prefix_pages = self.kv_manager.find_prefix(request.all_token_ids)
                request.num_computed_tokens = len(prefix_pages) * self.kv_manager.page_size
            remaining = request.num_tokens - request.num_computed_tokens
            if remaining <= 0:
                return None
            threshold = cfg.long_prefill_token_threshold
            if 0 < threshold < remaining:
                remaining = threshold
            num_tokens = min(remaining, token_budget)
            if not self.kv_manager.allocate_slots(request.request_id, num_tokens, prefix_pages):
                if prefix_pages:
                    request.num_computed_tokens = 0
                return None
            context = request.num_computed_tokens
            if from_waiting:
                new_reqs.append(
                    NewRequestData(
                        req_id=request.request_id,
                        prompt_token_ids=tuple(request.all_token_ids),
                        sampling_params=request.sampling_params,
                        num_computed_tokens=context,
                        num_output_tokens=request.num_output_tokens,
                    )
                )
            else:
                cached_ids.append(request.request_id)
                cached_tokens.append(tuple(request.all_token_ids[context : context + num_tokens]))
                cached_computed.append(context)
                cached_outputs.append(request.num_output_tokens)
            num_scheduled[request.request_id] = num_tokens
            return num_tokens, is_prefill

        # pass 1: running requests, in order; the first that cannot run stops the pass
        for request in list(self.running):
            if len(num_scheduled) >= cfg.max_num_seqs or token_budget <= 0:
                break
            if request.is_finished():
                continue
            scheduled = try_schedule(request, from_waiting=False)
            if scheduled is None:
                break
            num_tokens, is_prefill = scheduled
            if is_prefill:
                partial += 1
                long_partial += int(self._is_long_prefill(request))
            token_budget -= num_tokens

        # pass 2: waiting requests, first come first served
        skipped: list[Request] = []
        while self.waiting and len(num_scheduled) < cfg.max_num_seqs and token_budget > 0:
            request = self.waiting.popleft()
            scheduled = try_schedule(request, from_waiting=True)
            if scheduled is None:
                if self._is_prefill(request) and not self._can_schedule_partial_prefill(
                    request, partial, long_partial
                ):
                    skipped.append(request)  # blocked only by the prefill limit: try the next one
                    continue
                self.waiting.appendleft(request)
                break
            num_tokens, is_prefill = scheduled
            request.status = RequestStatus.RUNNING
            self.running.append(request)
            if is_prefill:
                partial += 1
                long_partial += int(self._is_long_prefill(request))
            token_budget -= num_tokens
        for request in reversed(skipped):
            self.waiting.appendleft(request)

        total = sum(num_scheduled.values())
        if total == 0 and not self.finished_req_ids:
            if self.has_unfinished_requests():
                return None
        finished = frozenset(self.finished_req_ids)
        self.finished_req_ids.clear()
        return SchedulerOutput(
            scheduled_new_reqs=tuple(new_reqs),
            scheduled_cached_reqs=CachedRequestData(
                req_ids=tuple(cached_ids),
                new_token_ids=tuple(cached_tokens),
                num_computed_tokens=tuple(cached_computed),
                num_output_tokens=tuple(cached_outputs),
            ),
            num_scheduled_tokens=num_scheduled,
            total_num_scheduled_tokens=total,
            finished_req_ids=finished,
            preempted_req_ids=tuple(preempted),
            step_id=self.step_id,
        )

    # ---- planning a step before the one in front has been read -----------------------------------
    def schedule_ahead(self, in_flight: SchedulerOutput) -> SchedulerOutput | None:
        """The plan of the step after ``in_flight``, made while ``in_flight`` still runs, or ``None``
        when that step is better planned once its tokens are in.

        What ``in_flight`` leaves behind is known except for the values of the tokens it samples:
        every request in it will have its scheduled tokens computed, and one that reaches the end
        of its tokens there will have one more token.  So the running requests can be served as
        ``schedule()`` would serve them, in order and under the same limits: the next portion of
        a prompt, or the one token in flight (its id is taken from the sampler's output on the
        device), unless the request ends by length with it.  The one thing not known is a stop
        token; a request that turns out to have stopped has its extra token dropped by
        ``update_from_outputs``.  Nothing here admits or preempts: with a request waiting that
        could be admitted, or pages that cannot be had, the answer is ``None``."""
        cfg = self.config
        if not self.running or in_flight.preempted_req_ids:
            return None
        if self.waiting and len(self.running) < cfg.max_num_seqs:
            return None
        scheduled_now = in_flight.num_scheduled_tokens
        max_model_len = self.kv_manager.max_model_len
        threshold = cfg.long_prefill_token_threshold
        token_budget = cfg.max_num_scheduled_tokens
        partial = long_partial = 0
        ids: list[str] = []
        tokens: list[tuple[int, ...]] = []
        computed: list[int] = []
        outputs: list[int] = []
        num_scheduled: dict[str, int] = {}
        pending: set[str] = set()
        for request in self.running:
            if len(num_scheduled) >= cfg.max_num_seqs or token_budget <= 0:
                break
            if request.is_finished():
                return None
            done = request.num_computed_tokens + scheduled_now.get(request.request_id, 0)
            samples = request.request_id in scheduled_now and done >= request.num_tokens
            if samples and (request.num_output_tokens + 1 >= request.max_tokens
                            or request.num_tokens + 1 >= max_model_len):
                continue                          # ends by length with the token in flight
            is_prefill = done < request.num_prompt_tokens
            if is_prefill:
                if not self._can_schedule_partial_prefill(request, partial, long_partial):
                    break                         # as in schedule(): the requests behind it wait too
                partial += 1
                long_partial += int(self._is_long_prefill(request))
            remaining = request.num_tokens + int(samples) - done
            if remaining <= 0 or (samples and remaining != 1):
                return None
            if 0 < threshold < remaining:
                remaining = threshold
            count = min(remaining, token_budget)
            # asking again for a page that is already there is harmless, so a refusal half-way
            # leaves nothing to undo
            if not self.kv_manager.allocate_slots(request.request_id, count):
                return None
            ids.append(request.request_id)
            tokens.append(() if samples else tuple(request.all_token_ids[done : done + count]))
            computed.append(done)
            outputs.append(request.num_output_tokens + int(samples))
            num_scheduled[request.request_id] = count
            if samples:
                pending.add(request.request_id)
            token_budget -= count
        if not num_scheduled:
            return None
        finished = frozenset(self.finished_req_ids)
        self.finished_req_ids.clear()
        return SchedulerOutput(
            scheduled_cached_reqs=CachedRequestData(
                req_ids=tuple(ids),
                new_token_ids=tuple(tokens),
                num_computed_tokens=tuple(computed),
                num_output_tokens=tuple(outputs),
            ),
            num_scheduled_tokens=num_scheduled,
            total_num_scheduled_tokens=sum(num_scheduled.values()),
            finished_req_ids=finished,
            step_id=self.step_id + 1,
            pending_token_req_ids=frozenset(pending),
        )

    # ---- after the step ----------------------------------------------------------------------------
    def update_from_outputs(
        self,
        scheduler_output: SchedulerOutput,
        sampled_token_ids: Mapping[str, int],
        *,
        stop_token_ids: set[int] | None = None,
    ) -> SchedulerUpdateResult:
        step_outputs: list[RequestStepOutput] = []
        finished_requests: list[FinishedRequestState] = []
        max_model_len = self.kv_manager.max_model_len
        for request_id, num_tokens in scheduler_output.num_scheduled_tokens.items():
            request = self.requests.get(request_id)
            if request is None:
                if request_id in scheduler_output.pending_token_req_ids:
                    continue   # planned ahead, then found to have stopped: its extra token is dropped
                raise KeyError(request_id)
            request.num_computed_tokens += num_tokens
            self.kv_manager.register_full_pages(request_id, request.all_token_ids)
            sampled: int | None = None
            finished = False
            reason: FinishReason | None = None
            if request.num_computed_tokens >= request.num_tokens:
                sampled = int(sampled_token_ids[request_id])
                request.append_output_token_id(sampled)
                if stop_token_ids is not None and sampled in stop_token_ids:
                    request.mark_finished(RequestStatus.FINISHED_STOPPED)
                elif request.num_output_tokens >= request.max_tokens:
                    request.mark_finished(RequestStatus.FINISHED_LENGTH_CAPPED)
                elif request.num_tokens >= max_model_len:
                    request.mark_finished(RequestStatus.FINISHED_LENGTH_CAPPED)
                if request.is_finished():
                    finished = True
                    reason = request.get_finished_reason()
                    finished_requests.append(self._free_finished_request(request))
                else:
                    request.status = RequestStatus.RUNNING
            else:
                request.status = RequestStatus.RUNNING
            step_outputs.append(RequestStepOutput(request_id, sampled, finished, reason))
        self.step_id += 1
        return SchedulerUpdateResult(tuple(step_outputs), tuple(finished_requests))

    # ---- helpers ---------------------------------------------------------------------------------
    @staticmethod
    def _is_prefill(request: Request) -> bool:
        return request.num_computed_tokens < request.num_prompt_tokens

    def _can_schedule_partial_prefill(self, request: Request, partial: int, long_partial: int) -> bool:
        if partial >= self.config.max_num_partial_prefills:
            return False
        return not (
            self._is_long_prefill(request) and long_partial >= self.config.max_long_partial_prefills
        )

    def _is_long_prefill(self, request: Request) -> bool:
        threshold = self.config.long_prefill_token_threshold
        return threshold > 0 and request.num_prompt_tokens >= threshold


__all__ = [
    "CachedRequestData",
    "FinishedRequestState",
    "NewRequestData",
    "RequestStepOutput",
    "Scheduler",
    "SchedulerNoProgressState",
    "SchedulerOutput",
    "SchedulerUpdateResult",
]
