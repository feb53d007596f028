"""Chat messages -> token ids: the folder's template is rendered with its own special tokens
(the beginning-of-text token included) and a template that cannot be rendered is an error.
Behaviour to match: the reference hands the messages to its tokenizer's chat template with the
generation prompt added (kvcore/utils/tokenizer.py:37-71, 96-114)."""
from __future__ import annotations

import json

import pytest

from kvcore_b200.utils.tokenizer import (ChatTemplateError, TokenizerManager, TokenizerUnavailable,
                                         render_chat_template)

tokenizers = pytest.importorskip("tokenizers")

SPECIALS = ["<|begin_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>", "<|end_of_text|>"]
WORDS = ["system", "user", "assistant", "be", "brief", "hello", "there", "what", "is", "two", "plus", "four", "\n\n"]

# a template in the manner of Llama 3 chat models: the text starts with the beginning-of-text token,
# every message is a header naming the role, a blank line, the trimmed content and an end-of-turn
# token; an unknown role stops the rendering; the generation prompt is an open assistant header
TEMPLATE = """{{ bos_token }}
{%- for message in messages %}
    {%- if message['role'] not in ['system', 'user', 'assistant'] %}
        {{- raise_exception('unknown role ' + message['role']) }}
    {%- endif %}
    {{- '<|start_header_id|>' + message['role'] + '<|end_header_id|>\n\n' + message['content'] | trim + '<|eot_id|>' }}
{%- endfor %}
{%- if add_generation_prompt %}
    {{- '<|start_header_id|>assistant<|end_header_id|>\n\n' }}
{%- endif %}
"""


def write_tokenizer(folder, template=TEMPLATE, *, bos="<|begin_of_text|>"):
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import WhitespaceSplit

    vocab = {word: index for index, word in enumerate(SPECIALS + ["[UNK]"] + WORDS)}
    tokenizer = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
    tokenizer.pre_tokenizer = WhitespaceSplit()
    tokenizer.add_special_tokens(SPECIALS)
    folder.mkdir(parents=True, exist_ok=True)
    tokenizer.save(str(folder / "tokenizer.json"))
    config = {"bos_token": bos, "eos_token": {"content": "<|eot_id|>"}}
    if template is not None:
        config["chat_template"] = template
    (folder / "tokenizer_config.json").write_text(json.dumps(config))
    return vocab


MESSAGES = [{"role": "system", "content": "be brief"}, {"role": "user", "content": " what is two plus four "}]


def test_messages_become_the_exact_ids_of_the_rendered_template(tmp_path):
    vocab = write_tokenizer(tmp_path / "m")
    manager = TokenizerManager(tmp_path / "m")
    text = manager.render_messages(MESSAGES)
    assert text == ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nbe brief<|eot_id|>"
                    "<|start_header_id|>user<|end_header_id|>\n\nwhat is two plus four<|eot_id|>"
                    "<|start_header_id|>assistant<|end_header_id|>\n\n")
    ids = manager.encode_messages(MESSAGES)
    v = vocab
    header = lambda role: [v["<|start_header_id|>"], v[role], v["<|end_header_id|>"]]
    assert ids == ([v["<|begin_of_text|>"]] + header("system") + [v["be"], v["brief"], v["<|eot_id|>"]]
                   + header("user") + [v["what"], v["is"], v["two"], v["plus"], v["four"], v["<|eot_id|>"]]
                   + header("assistant"))
    assert ids[0] == v["<|begin_of_text|>"] and ids.count(v["<|begin_of_text|>"]) == 1
    assert manager.get_stop_token_ids() == {v["<|eot_id|>"]}
    without_prompt = manager.encode_messages(MESSAGES, add_generation_prompt=False)
    assert without_prompt == ids[: -3]


def test_a_template_that_fails_raises_instead_of_changing_the_prompt(tmp_path):
    write_tokenizer(tmp_path / "bad", template="{{ bos_token }}{% for m in messages %}{{ m.nothing.here }}{% endfor %}")
    with pytest.raises(ChatTemplateError, match="could not be rendered"):
        TokenizerManager(tmp_path / "bad").encode_messages(MESSAGES)
    with pytest.raises(ChatTemplateError, match="unknown role tool"):
        render_chat_template(TEMPLATE, [{"role": "tool", "content": "x"}], bos_token="<s>")
    write_tokenizer(tmp_path / "none", template=None)
    with pytest.raises(ChatTemplateError, match="no chat template"):
        TokenizerManager(tmp_path / "none").encode_messages(MESSAGES)


def test_messages_are_checked_like_the_reference_checks_them(tmp_path):
    write_tokenizer(tmp_path / "m")
    manager = TokenizerManager(tmp_path / "m")
    with pytest.raises(ValueError, match="roles"):
        manager.encode_messages([{"role": "tool", "content": "x"}])
    with pytest.raises(TypeError, match="plain string"):
        manager.encode_messages([{"role": "user", "content": ["x"]}])


def test_template_helpers_are_there():
    text = render_chat_template("{{ messages | tojson }}|{{ strftime_now('%Y') | length }}|{{ eos_token }}",
                                [{"role": "user", "content": "é"}], eos_token="</s>")
    assert text == '[{"role": "user", "content": "é"}]|4|</s>'


def test_no_tokenizer_in_the_folder(tmp_path):
    manager = TokenizerManager(tmp_path)
    assert not manager.available and manager.decode([1, 2]) == ""
    with pytest.raises(TokenizerUnavailable):
        manager.encode_messages(MESSAGES)
