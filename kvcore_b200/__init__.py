"""kvcore_b200: a single-GPU inference engine for the Llama 3 decoder on NVIDIA B200."""
from .config import (
    CacheConfig,
    DeviceConfig,
    KVCoreConfig,
    LoadConfig,
    ModelConfig,
    SchedulerConfig,
)
from .sampling import SamplingParams

__version__ = "0.1.0"


def __getattr__(name: str):
    # the entry point pulls in torch-heavy modules; import it on first use
    if name in ("LLMEngine", "GenerationRequest", "GenerationOutput"):
        from .engine import llm_engine

        return getattr(llm_engine, name)
    raise AttributeError(name)


__all__ = [
    "CacheConfig",
    "DeviceConfig",
    "GenerationOutput",
    "GenerationRequest",
    "KVCoreConfig",
    "LLMEngine",
    "LoadConfig",
    "ModelConfig",
    "SamplingParams",
    "SchedulerConfig",
]
