"""Offline batch entry point: ``LLMEngine(config).generate(requests)``.

Surface as the reference's (kvcore/entry/llm_engine.py:15-107): ``GenerationRequest``,
``GenerationOutput``, ``add_request``, ``step``, ``generate``, and a RuntimeError when the
engine makes no progress.  A request here may carry ``prompt_token_ids`` instead of chat
``messages``; the tokenizer is optional.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

from ..config.engine_config import KVCoreConfig
from ..sampling.params import SamplingParams
from .engine_core import EngineCore, EngineCoreOutputs
from .runner import ModelRunner

logger = logging.getLogger("kvcore_b200.llm_engine")


@dataclass(frozen=True)
class GenerationRequest:
    request_id: str
    sampling_params: SamplingParams
    prompt_token_ids: tuple[int, ...] | None = None
    messages: tuple[Mapping[str, Any], ...] | None = None


@dataclass(frozen=True)
class GenerationOutput:
    request_id: str
    output_text: str
    output_token_ids: tuple[int, ...]
    finish_reason: str | None


class LLMEngine:
    def __init__(self, kvcore_config: KVCoreConfig, *, model_runner: ModelRunner | None = None) -> None:
        self.engine_core = EngineCore(kvcore_config, model_runner=model_runner)

    def add_request(
        self,
        request_id: str,
        sampling_params: SamplingParams,
        *,
        prompt_token_ids: Sequence[int] | None = None,
        messages: Sequence[Mapping[str, Any]] | None = None,
    ) -> None:
        self.engine_core.add_request(
            request_id, sampling_params, prompt_token_ids=prompt_token_ids, messages=messages
        )

    def step(self) -> EngineCoreOutputs:
        return self.engine_core.step()

    def generate(
        self, requests: Sequence[GenerationRequest | Mapping[str, Any]]
    ) -> list[GenerationOutput]:
        normalized = [self._normalize_request(request) for request in requests]
        for request in normalized:
            self.add_request(
                request.request_id,
                request.sampling_params,
                prompt_token_ids=request.prompt_token_ids,
                messages=request.messages,
            )
        while self.engine_core.has_unfinished_requests():
            step_output = self.step()
            if not step_output.request_outputs and self.engine_core.has_unfinished_requests():
                raise RuntimeError(
                    "Engine made no scheduling progress while requests are still unfinished. "
                    "This usually means the KV block budget is too small."
                )
        outputs: list[GenerationOutput] = []
        tokenizer = self.engine_core.tokenizer_manager
        for request in normalized:
            finished = self.engine_core.take_finished_output(request.request_id)
            if finished is None:
                continue
            outputs.append(
                GenerationOutput(
                    request_id=request.request_id,
                    output_text=tokenizer.decode(finished.output_token_ids),
                    output_token_ids=finished.output_token_ids,
                    finish_reason=None if finished.finish_reason is None else finished.finish_reason.value,
                )
            )
        return outputs

    @staticmethod
    def _normalize_request(request: GenerationRequest | Mapping[str, Any]) -> GenerationRequest:
        if isinstance(request, GenerationRequest):
            return request
        params = request["sampling_params"]
        if not isinstance(params, SamplingParams):
            params = SamplingParams(**dict(params))
        ids = request.get("prompt_token_ids")
        messages = request.get("messages")
        return GenerationRequest(
            request_id=str(request["request_id"]),
            sampling_params=params,
            prompt_token_ids=None if ids is None else tuple(int(t) for t in ids),
            messages=None if messages is None else tuple(messages),
        )


__all__ = ["GenerationOutput", "GenerationRequest", "LLMEngine"]
