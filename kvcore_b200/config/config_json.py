"""Reading a model folder's config.json: shared by every architecture's parser and the registry."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine refuses."""


def read_config_json(folder: str | Path) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in model folder {str(folder)!r}")
    with path.open("r", encoding="utf-8") as handle:
        raw = json.load(handle)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return raw


__all__ = ["ConfigError", "read_config_json"]
