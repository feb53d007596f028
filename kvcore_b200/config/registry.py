"""One registry from an architecture's name to how its model is described.

The reference keys its registry by ``model_type`` and maps to a model class
(kvcore/model/model_loader/default_loader.py:32-36, 64-70).  Here the value is a function
from the raw config.json dict to a ``ModelSpec``; the generic builder assembles the model
from that.  The key is ``architectures[0]`` of config.json, with ``model_type`` as a fallback.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from .config_json import ConfigError, read_config_json
from .model_spec import ModelSpec

SpecFactory = Callable[[Mapping[str, Any]], ModelSpec]


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    spec_from_config: SpecFactory
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, ArchitectureEntry] = {}


def register_architecture(
    name: str,
    spec_from_config: SpecFactory,
    *,
    model_types: tuple[str, ...] = (),
    replace: bool = False,
) -> None:
    """Add an architecture: ``spec_from_config(config_json_dict) -> ModelSpec``."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, spec_from_config, tuple(model_types))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(raw: Mapping[str, Any]) -> ArchitectureEntry:
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = raw.get("model_type")
    if model_type is not None:
        for entry in _ARCHITECTURES.values():
            if model_type in entry.model_types:
                return entry
    raise ConfigError(
        f"unsupported architecture: architectures={list(names)!r}, model_type={model_type!r}; "
        f"supported: {', '.join(registered_architectures())}"
    )


def model_spec_from_config(raw: Mapping[str, Any]) -> ModelSpec:
    return resolve_architecture(raw).spec_from_config(raw)


def model_spec_from_folder(folder: str | Path) -> ModelSpec:
    return model_spec_from_config(read_config_json(folder))


def _register_stock_architectures() -> None:
    from .llama import LlamaConfig

    register_architecture(
        "LlamaForCausalLM",
        lambda raw: LlamaConfig.from_dict(raw).to_model_spec(),
        model_types=("llama",),
    )


_register_stock_architectures()

__all__ = [
    "ArchitectureEntry",
    "model_spec_from_config",
    "model_spec_from_folder",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
    "unregister_architecture",
]
