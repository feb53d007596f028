"""Optional text front end: token ids are the engine's native input.

The reference always loads a tokenizer and renders chat messages through its template
(kvcore/utils/tokenizer.py:15-114).  Here a tokenizer is used only when the model folder
holds ``tokenizer.json`` and the ``tokenizers`` package can be imported; requests may always
carry ``prompt_token_ids`` instead, and outputs always carry token ids.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Sequence


class TokenizerUnavailable(RuntimeError):
    pass


class TokenizerManager:
    def __init__(self, folder: str | Path) -> None:
        self.folder = Path(folder)
        self._tokenizer = None
        self._chat_template: str | None = None
        self._eos_ids: set[int] = set()
        path = self.folder / "tokenizer.json"
        if path.is_file():
            try:
                from tokenizers import Tokenizer  # type: ignore

                self._tokenizer = Tokenizer.from_file(str(path))
            except Exception:  # missing package or unreadable file: run on token ids only
                self._tokenizer = None
        config_path = self.folder / "tokenizer_config.json"
        if config_path.is_file():
            try:
                with config_path.open("r", encoding="utf-8") as handle:
                    config = json.load(handle)
                self._chat_template = config.get("chat_template")
                eos = config.get("eos_token")
                if isinstance(eos, dict):
                    eos = eos.get("content")
                if eos and self._tokenizer is not None:
                    token_id = self._tokenizer.token_to_id(eos)
                    if token_id is not None:
                        self._eos_ids.add(int(token_id))
            except (OSError, json.JSONDecodeError):
                pass

    @property
    def available(self) -> bool:
        return self._tokenizer is not None

    def get_stop_token_ids(self) -> set[int]:
        return set(self._eos_ids)

    def encode_text(self, text: str) -> list[int]:
        if self._tokenizer is None:
            raise TokenizerUnavailable(
                f"no usable tokenizer in {str(self.folder)!r}: give prompt_token_ids instead of text"
            )
        return list(self._tokenizer.encode(text, add_special_tokens=False).ids)

    def encode_messages(self, messages: Sequence[Mapping[str, Any]]) -> list[int]:
        """Render chat messages with the folder's template when jinja2 is present, else
        join their contents with newlines; then encode."""
        if self._tokenizer is None:
            raise TokenizerUnavailable(
                f"no usable tokenizer in {str(self.folder)!r}: give prompt_token_ids instead of messages"
            )
        text = None
        if self._chat_template:
            try:
                import jinja2  # type: ignore

                template = jinja2.Environment().from_string(self._chat_template)
                text = template.render(messages=list(messages), add_generation_prompt=True, bos_token="")
            except Exception:
                text = None
        if text is None:
            text = "\n".join(str(message.get("content", "")) for message in messages)
        return self.encode_text(text)

    def decode(self, token_ids: Sequence[int]) -> str:
        if self._tokenizer is None:
            return ""
        return self._tokenizer.decode(list(token_ids), skip_special_tokens=True)


__all__ = ["TokenizerManager", "TokenizerUnavailable"]
