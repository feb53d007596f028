"""Configuration: engine-level settings, architecture descriptions and the registry."""
from .engine_config import (
    CacheConfig,
    DeviceConfig,
    KVCoreConfig,
    LoadConfig,
    ModelConfig,
    SchedulerConfig,
    normalize_dtype_name,
)
from .config_json import ConfigError, read_config_json
from .llama import LlamaConfig, RopeScaling
from .model_spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, default_schedule
from .registry import (
    model_spec_from_config,
    model_spec_from_folder,
    register_architecture,
    registered_architectures,
    resolve_architecture,
    unregister_architecture,
)

__all__ = [
    "CacheConfig",
    "ConfigError",
    "DeviceConfig",
    "KVCoreConfig",
    "LayerSpec",
    "LlamaConfig",
    "LoadConfig",
    "ModelConfig",
    "ModelSpec",
    "PartSpec",
    "RopeScaling",
    "ScheduleEntry",
    "SchedulerConfig",
    "default_schedule",
    "model_spec_from_config",
    "model_spec_from_folder",
    "normalize_dtype_name",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
