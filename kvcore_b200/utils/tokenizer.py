"""Optional text front end: token ids are the engine's native input.

The reference always loads a tokenizer and renders chat messages through its template
(kvcore/utils/tokenizer.py:15-114).  Here a tokenizer is used only when the model folder
holds ``tokenizer.json`` and the ``tokenizers`` package can be imported; requests may always
carry ``prompt_token_ids`` instead, and outputs always carry token ids.

Chat messages are rendered the way the reference's tokenizer renders them: the folder's
``chat_template`` is a Jinja template evaluated in a sandboxed environment with block
trimming, given ``messages``, ``add_generation_prompt``, ``bos_token`` and ``eos_token`` (from
``tokenizer_config.json``) and the helpers ``raise_exception``, ``strftime_now`` and ``tojson``;
the rendered text, which names its special tokens itself (a Llama 3 template starts with
``{{ bos_token }}``), is encoded without adding any.  A template that cannot be rendered is an
error, never a silently different prompt.
"""
from __future__ import annotations

import json
from datetime import datetime
from pathlib import Path
from typing import Any, Mapping, Sequence


class TokenizerUnavailable(RuntimeError):
    pass


class ChatTemplateError(ValueError):
    """The folder's chat template is missing or could not be rendered for these messages."""


_ROLES = ("system", "user", "assistant")


def _token_text(value: Any) -> str:
    """``bos_token`` / ``eos_token`` of tokenizer_config.json: a string, or a mapping with ``content``."""
    if isinstance(value, Mapping):
        value = value.get("content")
    return value if isinstance(value, str) else ""


def normalize_messages(messages: Sequence[Mapping[str, Any]]) -> list[dict[str, str]]:
    """Messages as the reference accepts them (kvcore/utils/tokenizer.py:96-114): one of three
    roles and a plain string each."""
    out = []
    for message in messages:
        role, content = message.get("role"), message.get("content")
        if role not in _ROLES:
            raise ValueError(f"messages must use one of the roles {', '.join(map(repr, _ROLES))}, got {role!r}")
        if not isinstance(content, str):
            raise TypeError(f"message content must be a plain string, got {type(content)!r}")
        out.append({"role": role, "content": content})
    return out


def render_chat_template(template: str, messages: Sequence[Mapping[str, Any]], *, bos_token: str = "",
                         eos_token: str = "", add_generation_prompt: bool = True) -> str:
    """The text a chat template makes of ``messages``; raises ``ChatTemplateError`` if it cannot."""
    try:
        import jinja2
        from jinja2.sandbox import ImmutableSandboxedEnvironment
    except ImportError as error:  # pragma: no cover - jinja2 ships with the image
        raise ChatTemplateError(f"rendering a chat template needs jinja2: {error}") from error

    def raise_exception(message: str):
        raise jinja2.exceptions.TemplateError(message)

    def tojson(value, ensure_ascii=False, indent=None, separators=None, sort_keys=False):
        return json.dumps(value, ensure_ascii=ensure_ascii, indent=indent, separators=separators,
                          sort_keys=sort_keys)

    environment = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
    environment.filters["tojson"] = tojson
    environment.globals["raise_exception"] = raise_exception
    environment.globals["strftime_now"] = lambda pattern: datetime.now().strftime(pattern)
    try:
        return environment.from_string(template).render(
            messages=list(messages), add_generation_prompt=add_generation_prompt,
            bos_token=bos_token, eos_token=eos_token)
    except jinja2.exceptions.TemplateError as error:
        raise ChatTemplateError(f"the chat template could not be rendered: {error}") from error


class TokenizerManager:
    def __init__(self, folder: str | Path) -> None:
        self.folder = Path(folder)
        self._tokenizer = None
        self._chat_template: str | None = None
        self._bos_token = ""
        self._eos_token = ""
        self._eos_ids: set[int] = set()
        path = self.folder / "tokenizer.json"
        if path.is_file():
            try:
                from tokenizers import Tokenizer  # type: ignore
            except ImportError:      # no package: run on token ids only
                Tokenizer = None
            if Tokenizer is not None:
                self._tokenizer = Tokenizer.from_file(str(path))
        config_path = self.folder / "tokenizer_config.json"
        if config_path.is_file():
            with config_path.open("r", encoding="utf-8") as handle:
                config = json.load(handle)
            template = config.get("chat_template")
            if isinstance(template, list):      # several named templates: the one called "default"
                named = {item.get("name"): item.get("template") for item in template if isinstance(item, Mapping)}
                template = named.get("default")
            self._chat_template = template if isinstance(template, str) else None
            self._bos_token = _token_text(config.get("bos_token"))
            self._eos_token = _token_text(config.get("eos_token"))
            if self._eos_token and self._tokenizer is not None:
                token_id = self._tokenizer.token_to_id(self._eos_token)
                if token_id is not None:
                    self._eos_ids.add(int(token_id))
        template_file = self.folder / "chat_template.jinja"
        if self._chat_template is None and template_file.is_file():
            self._chat_template = template_file.read_text(encoding="utf-8")

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

    def render_messages(self, messages: Sequence[Mapping[str, Any]], *, add_generation_prompt: bool = True) -> str:
        if not self._chat_template:
            raise ChatTemplateError(
                f"{str(self.folder)!r} has no chat template: give prompt_token_ids instead of messages")
        return render_chat_template(self._chat_template, normalize_messages(messages),
                                    bos_token=self._bos_token, eos_token=self._eos_token,
                                    add_generation_prompt=add_generation_prompt)

    def encode_messages(self, messages: Sequence[Mapping[str, Any]], *, add_generation_prompt: bool = True) -> list[int]:
        """Render chat messages with the folder's template and encode the text as it stands (the
        template writes the special tokens, the beginning-of-text token included)."""
        if self._tokenizer is None:
            raise TokenizerUnavailable(
                f"no usable tokenizer in {str(self.folder)!r}: give prompt_token_ids instead of messages"
            )
        return self.encode_text(self.render_messages(messages, add_generation_prompt=add_generation_prompt))

    def decode(self, token_ids: Sequence[int]) -> str:
        if self._tokenizer is None:
            return ""
        return self._tokenizer.decode(list(token_ids), skip_special_tokens=True)


__all__ = ["ChatTemplateError", "TokenizerManager", "TokenizerUnavailable", "normalize_messages",
           "render_chat_template"]
