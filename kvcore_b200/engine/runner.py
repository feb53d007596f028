"""Model runner: builds the model and its cache, and turns a scheduler output into one
call of the step function followed by sampling.

Counterpart of the reference's runner (kvcore/model/model_runner.py:125-206 load and cache
set-up, 208-306 execute, 308-353 sample, 355-409 request bookkeeping; loader:
kvcore/model/model_loader/default_loader.py:44-96).  The runner keeps each live request's
token ids (prompt plus sampled tokens), so cached requests need not resend them; logits are
asked only for a request whose scheduled portion reaches the end of its known tokens.
"""
from __future__ import annotations

import logging
import time
from dataclasses import dataclass
from pathlib import Path

import torch

from .. import kernels as K
from ..cache.kv_manager import KVManager, group_entries
from ..config.engine_config import KVCoreConfig
from ..config.registry import model_spec_from_folder
from ..parts.model import DecoderModel, build_model
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model_weights
from ..weights.random_init import init_random_weights_
from .scheduler import SchedulerOutput
from .step import CacheStorage, StepEntry, StepFunction

logger = logging.getLogger("kvcore_b200.runner")

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def resolve_dtype(requested: str | None, stored: str | None) -> torch.dtype:
    """The compute dtype: what the user asked for, else what config.json names, else bfloat16."""
    from ..config.engine_config import normalize_dtype_name

    name = requested
    if name is None and stored is not None:
        try:
            name = normalize_dtype_name(stored)
        except ValueError:
            name = None  # e.g. float16 checkpoints run in bfloat16
    return _TORCH_DTYPES[name or "bfloat16"]


def load_model(config: KVCoreConfig) -> DecoderModel:
    """config.json -> registry -> parts on the device -> weights (files or seeded random)."""
    device = torch.device(config.device_config.device)
    K.require_device(device)
    folder = Path(config.model_config.model)
    spec = model_spec_from_folder(folder)
    dtype = resolve_dtype(config.model_config.dtype, spec.stored_dtype)
    started = time.perf_counter()
    model = build_model(spec, dtype=dtype, device=device)
    if config.load_config.random_weights:
        init_random_weights_(model, config.load_config.seed, config.load_config.init_std)
    else:
        load_model_weights(model, folder, strict=config.load_config.strict)
    logger.info("model %s loaded in %.2fs as %s", folder, time.perf_counter() - started, dtype)
    return model


@dataclass
class CachedRequestState:
    """Runner-side memory of a live request (reference: kvcore/model/input_batch.py:14-33)."""

    request_id: str
    token_ids: list[int]
    sampling_params: SamplingParams
    seed: int
    num_sampled: int = 0


@dataclass
class ModelRunnerOutput:
    req_ids: list[str]
    sampled_token_ids: list[list[int]]


@dataclass
class StepStats:
    """Host-side timings of the last step, in seconds (reference: model_runner.py:81-91)."""

    num_reqs: int = 0
    num_tokens: int = 0
    num_sampled: int = 0
    forward_sec: float = 0.0
    sample_sec: float = 0.0


@dataclass
class _PendingSample:
    logits: torch.Tensor | None
    req_ids: list[str]
    sampled_req_ids: list[str]


@dataclass
class SampleHandle:
    """Tokens that the device is sampling (or has sampled) and the host has not read yet.

    ``tokens`` (int32 on the device, one row per sampled request) can feed the next step before
    anyone has seen it; ``collect`` waits for ``ready`` and reads the pinned copy."""

    req_ids: list[str]
    states: list[CachedRequestState]
    tokens: torch.Tensor | None = None
    host: torch.Tensor | None = None
    ready: "torch.cuda.Event | None" = None

    def row_of(self, request_id: str) -> int | None:
        for row, state in enumerate(self.states):
            if state.request_id == request_id:
                return row
        return None


class ModelRunner:
    def __init__(self, config: KVCoreConfig, model: DecoderModel | None = None) -> None:
        self.config = config
        self.device = torch.device(config.device_config.device)
        self.model = model if model is not None else load_model(config)
        self.dtype = self.model.dtype
        spec = self.model.spec
        self.max_model_len = config.model_config.max_model_len or spec.max_position_embeddings
        self.page_size = config.cache_config.block_size
        self.max_num_seqs = config.scheduler_config.max_num_seqs
        self.max_num_tokens = config.scheduler_config.max_num_scheduled_tokens

        requirements = self.model.entry_requirements()
        self.groups, self.entry_group = group_entries(requirements)
        num_pages = self._decide_num_pages()
        self.kv_manager = KVManager(
            self.groups,
            num_pages=num_pages,
            page_size=self.page_size,
            max_num_seqs=self.max_num_seqs,
            max_model_len=self.max_model_len,
            # state that a mixer keeps per request cannot be taken over with the pages
            enable_prefix_caching=config.cache_config.enable_prefix_caching
            and not any(req.state_spec is not None for req in requirements),
            track_released_pages=config.cache_config.debug_fill_freed_pages is not None,
        )
        self.storage = CacheStorage(
            self.model,
            self.groups,
            self.entry_group,
            num_pages=num_pages,
            page_size=self.page_size,
            num_slots=self.max_num_seqs,
            dtype=self.dtype,
            device=self.device,
        )
        self.step_function = StepFunction(
            self.model,
            self.kv_manager,
            self.storage,
            max_num_tokens=self.max_num_tokens,
            max_num_seqs=self.max_num_seqs,
            use_cuda_graphs=not config.model_config.enforce_eager,
            fill_freed_pages=config.cache_config.debug_fill_freed_pages,
        )
        self.sampler = Sampler(self.device)
        self.requests: dict[str, CachedRequestState] = {}
        self._pending: _PendingSample | None = None
        self.last_stats = StepStats()
        # sampled tokens come back through pinned buffers in turn; two steps may be unread at once
        self._token_buffers: list[tuple[torch.Tensor, torch.cuda.Event]] = []
        self._token_turn = 0

    # ---- cache sizing ------------------------------------------------------------------------
    def bytes_per_page(self) -> list[int]:
        """Bytes one page id costs in each group: every plane of every entry of the group."""
        item = torch.empty((), dtype=self.dtype).element_size()
        return [
            len(group.entries) * group.elements_per_token * self.page_size * item
            for group in self.groups
        ]

    def _decide_num_pages(self) -> list[int]:
        """Pages per group: the configured count, else what fits in free device memory.

        The reference profiles a dummy forward to find the non-cache peak
        (model_runner.py:696-768); here weights are already resident, so the budget is the
        free memory times ``gpu_memory_utilization`` minus room for one step's activations,
        split over groups in proportion to their page cost, capped at what
        ``max_num_seqs`` full-length requests could ever use.
        """
        cache_cfg = self.config.cache_config
        if not self.groups:
            return []
        if cache_cfg.num_gpu_blocks is not None:
            return [cache_cfg.num_gpu_blocks] * len(self.groups)
        per_seq = -(-self.max_model_len // self.page_size)
        ceiling = self.max_num_seqs * per_seq + 1
        if self.device.type != "cuda":
            return [ceiling] * len(self.groups)
        free_bytes, _total = torch.cuda.mem_get_info(self.device)
        spec = self.model.spec
        item = torch.empty((), dtype=self.dtype).element_size()
        widest = max(spec.hidden_size * 8, spec.vocab_size)
        activation_bytes = self.max_num_tokens * widest * item * 4 + (512 << 20)
        budget = int(free_bytes * cache_cfg.gpu_memory_utilization) - activation_bytes
        costs = self.bytes_per_page()
        pages = max(budget // sum(costs), 0)
        if pages < per_seq + 1:
            raise RuntimeError(
                f"not enough device memory for the cache: room for {pages} pages per group, "
                f"one request of max_model_len {self.max_model_len} needs {per_seq + 1}"
            )
        return [int(min(pages, ceiling))] * len(self.groups)

    # ---- one step ------------------------------------------------------------------------------
    def execute_model(self, scheduler_output: SchedulerOutput, feed: SampleHandle | None = None) -> None:
        """Run the scheduled tokens; logits are kept for ``sample_tokens``.

        ``feed``: the handle of the step in front, when ``scheduler_output`` was planned before that
        step's tokens were read (its ``pending_token_req_ids``): those requests' tokens are taken
        from the sampler's output on the device."""
        if self._pending is not None:
            raise RuntimeError("execute_model called twice without sample_tokens")
        started = time.perf_counter()
        self.remove_requests(scheduler_output.finished_req_ids)
        self.remove_requests(scheduler_output.preempted_req_ids)
        for new in scheduler_output.scheduled_new_reqs:
            seed = new.sampling_params.seed
            self.requests[new.req_id] = CachedRequestState(
                request_id=new.req_id,
                token_ids=list(new.prompt_token_ids),
                sampling_params=new.sampling_params,
                seed=self.sampler.fresh_seed() if seed is None else int(seed),
                num_sampled=new.num_output_tokens,
            )
        cached = scheduler_output.scheduled_cached_reqs
        for req_id, new_tokens, computed in zip(
            cached.req_ids, cached.new_token_ids, cached.num_computed_tokens
        ):
            state = self.requests[req_id]
            known = len(state.token_ids)
            end = computed + len(new_tokens)
            if end > known:  # tokens the runner has not recorded itself
                state.token_ids.extend(new_tokens[known - computed :])

        entries: list[StepEntry] = []
        sampled_req_ids: list[str] = []
        req_ids: list[str] = []
        for req_id, num_tokens in scheduler_output.num_scheduled_tokens.items():
            state = self.requests[req_id]
            start = self.kv_manager.num_computed(req_id)
            end = start + num_tokens
            want: tuple[int, ...] = ()
            if end >= len(state.token_ids):
                want = (num_tokens - 1,)
                sampled_req_ids.append(req_id)
            if req_id in scheduler_output.pending_token_req_ids:
                row = None if feed is None else feed.row_of(req_id)
                if row is None or num_tokens != 1 or start != len(state.token_ids):
                    raise RuntimeError(f"request {req_id!r} was planned on a token that no step in flight samples")
                entries.append(StepEntry(req_id, (0,), want, fed_from=row))
            else:
                entries.append(StepEntry(req_id, state.token_ids[start:end], want))
            req_ids.append(req_id)
        feedback = feed.tokens if feed is not None and scheduler_output.pending_token_req_ids else None
        logits = self.step_function.step(entries, feedback) if entries else None
        self._pending = _PendingSample(logits, req_ids, sampled_req_ids)
        self.last_stats = StepStats(
            num_reqs=len(entries),
            num_tokens=scheduler_output.total_num_scheduled_tokens,
            num_sampled=len(sampled_req_ids),
            forward_sec=time.perf_counter() - started,
        )

    def launch_sampling(self) -> SampleHandle:
        """Start sampling from the logits of the last ``execute_model`` and start their copy to
        the host; returns at once."""
        if self._pending is None:
            raise RuntimeError("sample_tokens called without execute_model")
        pending, self._pending = self._pending, None
        started = time.perf_counter()
        states = [self.requests[r] for r in pending.sampled_req_ids]
        handle = SampleHandle(pending.req_ids, states)
        if states:
            handle.tokens = self.sampler.sample(
                pending.logits,
                [s.sampling_params for s in states],
                [s.seed for s in states],
                [s.num_sampled for s in states],
            )
            for state in states:
                state.num_sampled += 1
            if handle.tokens.device.type == "cuda":
                if len(self._token_buffers) < 4:
                    self._token_buffers.append((torch.empty(self.max_num_seqs, dtype=torch.int32, pin_memory=True),
                                                torch.cuda.Event()))
                buffer, event = self._token_buffers[self._token_turn % len(self._token_buffers)]
                self._token_turn += 1
                handle.host = buffer[: len(states)]
                handle.host.copy_(handle.tokens, non_blocking=True)
                event.record()
                handle.ready = event
            else:
                handle.host = handle.tokens
        self.last_stats.sample_sec = time.perf_counter() - started
        return handle

    def collect(self, handle: SampleHandle) -> ModelRunnerOutput:
        """Wait for the tokens of ``handle`` and record them in the requests' token lists."""
        sampled: dict[str, int] = {}
        if handle.states:
            if handle.ready is not None:
                handle.ready.synchronize()
            tokens = handle.host.tolist()
            # the step has finished (its tokens are here): anything its kernels reported is read
            # from host memory, without another round trip
            K.raise_on_status()
            for state, token in zip(handle.states, tokens):
                state.token_ids.append(int(token))
                sampled[state.request_id] = int(token)
        return ModelRunnerOutput(
            req_ids=handle.req_ids,
            sampled_token_ids=[[sampled[r]] if r in sampled else [] for r in handle.req_ids],
        )

    def sample_tokens(self) -> ModelRunnerOutput:
        return self.collect(self.launch_sampling())

    def remove_requests(self, request_ids) -> None:
        for request_id in request_ids:
            self.requests.pop(request_id, None)


__all__ = [
    "CachedRequestState",
    "ModelRunner",
    "ModelRunnerOutput",
    "SampleHandle",
    "StepStats",
    "load_model",
    "resolve_dtype",
]
