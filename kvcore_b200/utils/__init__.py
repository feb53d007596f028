"""Logging and the optional tokenizer front end."""
from .log import configure_logging, get_logger

__all__ = ["configure_logging", "get_logger"]
