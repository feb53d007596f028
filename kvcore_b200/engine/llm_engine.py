"""Offline batch entry point: ``LLMEngine(config).generate(requests)``.

The names a user of the reference knows are kept (kvcore/entry/llm_engine.py:15-107):
``GenerationRequest``, ``GenerationOutput``, ``LLMEngine.add_request / step / generate``, and a
RuntimeError when nothing can be scheduled while requests are unfinished.  Here a request may
bring ``prompt_token_ids`` instead of chat ``messages`` (the tokenizer is optional), and
``run`` yields the outputs of every step for callers that want tokens as they appear.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterator, Mapping, Sequence

from ..config.engine_config import KVCoreConfig
from ..sampling.params import SamplingParams
from .engine_core import EngineCore, EngineCoreOutputs, FinishedRequestOutput
from .runner import ModelRunner

NO_PROGRESS = ("Engine made no scheduling progress while requests are still unfinished: "
               "the cache has too few pages for what is waiting.")


@dataclass(frozen=True)
class GenerationRequest:
    request_id: str
    sampling_params: SamplingParams
    prompt_token_ids: tuple[int, ...] | None = None
    messages: tuple[Mapping[str, Any], ...] | None = None

    @classmethod
    def coerce(cls, item: "GenerationRequest | Mapping[str, Any]") -> "GenerationRequest":
        """A request as given by the caller: already one of these, or a mapping with
        ``request_id``, ``sampling_params`` (object or mapping) and a prompt in either form."""
        if isinstance(item, cls):
            return item
        params = item["sampling_params"]
        if not isinstance(params, SamplingParams):
            params = SamplingParams.from_mapping(params)
        ids, messages = item.get("prompt_token_ids"), item.get("messages")
        return cls(
            str(item["request_id"]),
            params,
            tuple(map(int, ids)) if ids is not None else None,
            tuple(messages) if messages is not None else None,
        )


@dataclass(frozen=True)
class GenerationOutput:
    request_id: str
    output_text: str
    output_token_ids: tuple[int, ...]
    finish_reason: str | None


class LLMEngine:
    def __init__(self, kvcore_config: KVCoreConfig, *, model_runner: ModelRunner | None = None) -> None:
        self.engine_core = EngineCore(kvcore_config, model_runner=model_runner)

    def add_request(self, request_id: str, sampling_params: SamplingParams, *,
                    prompt_token_ids: Sequence[int] | None = None,
                    messages: Sequence[Mapping[str, Any]] | None = None) -> None:
        self.engine_core.add_request(request_id, sampling_params,
                                     prompt_token_ids=prompt_token_ids, messages=messages)

    def step(self) -> EngineCoreOutputs:
        return self.engine_core.step()

    def abort(self, request_ids: Sequence[str] | None = None) -> list[GenerationOutput]:
        """End the given requests (all of them for ``None``) now; returns what they had generated."""
        return [self._as_output(finished) for finished in self.engine_core.abort_requests(request_ids)]

    def run(self) -> Iterator[EngineCoreOutputs]:
        """Steps until every admitted request has finished, yielding each step's outputs."""
        core = self.engine_core
        while core.has_unfinished_requests():
            outputs = core.step()
            if not outputs.request_outputs and core.has_unfinished_requests():
                raise RuntimeError(NO_PROGRESS)
            yield outputs

    def generate(self, requests: Sequence[GenerationRequest | Mapping[str, Any]]) -> list[GenerationOutput]:
        """Admits ``requests``, runs them to the end and returns their outputs in the given order."""
        batch = [GenerationRequest.coerce(item) for item in requests]
        for request in batch:
            self.add_request(request.request_id, request.sampling_params,
                             prompt_token_ids=request.prompt_token_ids, messages=request.messages)
        for _ in self.run():
            pass
        taken = (self.engine_core.take_finished_output(request.request_id) for request in batch)
        return [self._as_output(finished) for finished in taken if finished is not None]

    def _as_output(self, finished: FinishedRequestOutput) -> GenerationOutput:
        reason = finished.finish_reason
        return GenerationOutput(
            request_id=finished.request_id,
            output_text=self.engine_core.tokenizer_manager.decode(finished.output_token_ids),
            output_token_ids=finished.output_token_ids,
            finish_reason=reason.value if reason is not None else None,
        )


__all__ = ["GenerationOutput", "GenerationRequest", "LLMEngine"]
