"""Engine-level configuration: frozen dataclasses composed into one KVCoreConfig.

Mirrors the shape of the reference's configuration (kvcore/config.py:15-191): a model,
load, cache, scheduler and device sub-config under one top object, each validated in
``__post_init__``.  What differs: the model is described by a folder with config.json
(parsed by this package, no third-party config class), there is a single CUDA code path
(no attention-backend switch), and loading has a seeded random-weights mode.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path

_DTYPE_ALIASES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
    "float": "float32",
}


def normalize_dtype_name(name: str | None) -> str | None:
    """Map a user-facing dtype name onto "bfloat16" or "float32" (None stays None)."""
    if name is None:
        return None
    key = str(name).replace("torch.", "").lower()
    if key not in _DTYPE_ALIASES:
        raise ValueError(f"dtype must be one of {sorted(set(_DTYPE_ALIASES))}, got {name!r}")
    return _DTYPE_ALIASES[key]


@dataclass(frozen=True, slots=True)
class ModelConfig:
    """Which model to run (reference: kvcore/config.py:15-29).

    ``model`` is a folder holding config.json and safetensors weights.  ``dtype`` selects
    the kernel family: "bfloat16" (serving precision) or "float32" (true 32-bit everywhere).
    ``None`` takes the dtype named in config.json, else bfloat16.  ``enforce_eager`` turns off
    the CUDA graphs that decode-only steps otherwise replay.
    """

    model: str | Path
    dtype: str | None = None
    max_model_len: int | None = None
    enforce_eager: bool = False

    def __post_init__(self) -> None:
        if self.max_model_len is not None and self.max_model_len <= 0:
            raise ValueError(f"max_model_len must be positive, got {self.max_model_len}")
        object.__setattr__(self, "dtype", normalize_dtype_name(self.dtype))


@dataclass(frozen=True, slots=True)
class LoadConfig:
    """How weights are obtained (reference: kvcore/config.py:32-39).

    ``strict`` makes missing/unexpected/mis-shaped tensors an error.  ``random_weights``
    skips the safetensors files and draws every matrix from N(0, init_std) with ``seed``.
    """

    strict: bool = True
    random_weights: bool = False
    seed: int = 0
    init_std: float = 0.02

    def __post_init__(self) -> None:
        if self.init_std < 0:
            raise ValueError(f"init_std must be non-negative, got {self.init_std}")


@dataclass(frozen=True, slots=True)
class CacheConfig:
    """Paged cache sizing (reference: kvcore/config.py:42-59).

    ``block_size`` is the number of tokens a page holds.  ``num_gpu_blocks`` fixes the
    number of pages per cache group; when None the pool is sized from free device memory
    times ``gpu_memory_utilization``.  ``enable_prefix_caching`` (the reference's
    ``enable_caching``): requests whose prompts begin with the same full pages share them.
    ``debug_fill_freed_pages`` (a debugging aid, off by default): pages that nobody holds any more
    are overwritten before the next step runs, with zeros (``"zero"``; the reference zeroes every
    freshly allocated block, kvcore/model/model_runner.py:646-657) or with a large finite value
    (``"poison"``), so that a kernel that reads a position its request has not written shows in the
    logits.  The value is finite because the tensor-core kernels multiply whole value tiles with
    probabilities that are exactly zero at masked positions, and ``0 * NaN`` is not zero.  Not
    together with prefix caching, which reads freed pages on purpose.
    """

    block_size: int = 16
    num_gpu_blocks: int | None = None
    gpu_memory_utilization: float = 0.9
    enable_prefix_caching: bool = False
    debug_fill_freed_pages: str | None = None

    def __post_init__(self) -> None:
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks <= 0:
            raise ValueError(f"num_gpu_blocks must be positive, got {self.num_gpu_blocks}")
        if not 0 < self.gpu_memory_utilization <= 1:
            raise ValueError(
                f"gpu_memory_utilization must be in (0, 1], got {self.gpu_memory_utilization}"
            )
        if self.debug_fill_freed_pages not in (None, "zero", "poison"):
            raise ValueError(
                f"debug_fill_freed_pages must be None, 'zero' or 'poison', got {self.debug_fill_freed_pages!r}"
            )
        if self.debug_fill_freed_pages is not None and self.enable_prefix_caching:
            raise ValueError("debug_fill_freed_pages cannot be combined with enable_prefix_caching: "
                             "prefix reuse reads pages after their last holder let go of them")


@dataclass(frozen=True, slots=True)
class SchedulerConfig:
    """Continuous-batching limits (reference: kvcore/config.py:62-92).

    ``preempt_on_deadlock``: when every running request is blocked on pages and nothing
    can be scheduled, free the youngest running request and queue it for recompute instead
    of reporting no progress (the reference only reports; kvcore/sched/scheduler.py:263-273).
    ``run_ahead``: keep one step in flight: a batch in steady decoding has its next step planned
    and launched before the tokens of the current one are read (not in the reference).
    """

    max_num_seqs: int = 8
    max_num_scheduled_tokens: int = 512
    max_num_partial_prefills: int = 1
    max_long_partial_prefills: int = 1
    long_prefill_token_threshold: int = 0
    preempt_on_deadlock: bool = True
    run_ahead: bool = True

    def __post_init__(self) -> None:
        for name in (
            "max_num_seqs",
            "max_num_scheduled_tokens",
            "max_num_partial_prefills",
            "max_long_partial_prefills",
        ):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        if self.long_prefill_token_threshold < 0:
            raise ValueError(
                "long_prefill_token_threshold must be non-negative, "
                f"got {self.long_prefill_token_threshold}"
            )


@dataclass(frozen=True, slots=True)
class DeviceConfig:
    """Target device (reference: kvcore/config.py:159-161).  Only CUDA devices run."""

    device: str = "cuda:0"


@dataclass(frozen=True, slots=True)
class KVCoreConfig:
    """Top-level configuration (reference: kvcore/config.py:164-191)."""

    model_config: ModelConfig
    load_config: LoadConfig = field(default_factory=LoadConfig)
    cache_config: CacheConfig = field(default_factory=CacheConfig)
    scheduler_config: SchedulerConfig = field(default_factory=SchedulerConfig)
    device_config: DeviceConfig = field(default_factory=DeviceConfig)


__all__ = [
    "CacheConfig",
    "DeviceConfig",
    "KVCoreConfig",
    "LoadConfig",
    "ModelConfig",
    "SchedulerConfig",
    "normalize_dtype_name",
]
