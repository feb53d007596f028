"""Logging under the ``kvcore_b200`` logger; default level WARNING, overridable with the
``KVCORE_LOG_LEVEL`` environment variable (reference: kvcore/utils/log.py:12-59)."""
from __future__ import annotations

import logging
import os
import sys

_ROOT = "kvcore_b200"
_configured = False


def configure_logging(level: str | int | None = None, *, force: bool = False) -> None:
    global _configured
    if _configured and not force:
        return
    if level is None:
        level = os.environ.get("KVCORE_LOG_LEVEL", "WARNING")
    if isinstance(level, str):
        level = getattr(logging, level.upper(), logging.WARNING)
    root = logging.getLogger(_ROOT)
    root.setLevel(level)
    if force:
        for handler in list(root.handlers):
            root.removeHandler(handler)
    if not root.handlers:
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
        root.addHandler(handler)
    root.propagate = False
    _configured = True


def get_logger(name: str) -> logging.Logger:
    configure_logging()
    return logging.getLogger(name if name.startswith(_ROOT) else f"{_ROOT}.{name}")


__all__ = ["configure_logging", "get_logger"]
