"""Configuration: config.json keys, defaults, refusals, the registry and the model description."""
from __future__ import annotations

import json

import pytest
import torch

from kvcore_b200.config import (
    CacheConfig, ConfigError, KVCoreConfig, LlamaConfig, ModelConfig, SchedulerConfig,
    model_spec_from_config, model_spec_from_folder, register_architecture, registered_architectures,
    unregister_architecture,
)
from kvcore_b200.config.model_spec import ModelSpec, PartSpec, ScheduleEntry
from kvcore_b200.parts.rope import rope_inverse_frequencies

import plain_llama
import replay_cases as rc


def test_llama_keys_and_defaults():
    cfg = LlamaConfig.from_dict(dict(vocab_size=100, hidden_size=64, intermediate_size=128,
                                     num_hidden_layers=2, num_attention_heads=4))
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 10000.0
    assert cfg.rope_scaling.rope_type == "default"
    assert not cfg.tie_word_embeddings and not cfg.attention_bias and not cfg.mlp_bias
    assert cfg.eos_token_ids == ()


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_tiny_configs_parse(name):
    raw = rc.TINY_CONFIGS[name]
    cfg = LlamaConfig.from_dict(raw)
    spec = cfg.to_model_spec()
    assert len(spec.layers) == raw["num_hidden_layers"] == len(spec.schedule)
    assert spec.layers[0].mixer.params["head_dim"] == plain_llama.head_dim_of(raw)
    assert spec.layers[0].mixer.params["scale"] == plain_llama.head_dim_of(raw) ** -0.5
    assert spec.layers[1].norms["mixer_norm"].params["eps"] == raw["rms_norm_eps"]
    assert (spec.lm_head.params["tied_to"] is not None) == raw["tie_word_embeddings"]


def test_rope_parameters_and_legacy_scaling_agree():
    base = dict(vocab_size=10, hidden_size=32, intermediate_size=8, num_hidden_layers=1, num_attention_heads=2)
    scaling = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                   original_max_position_embeddings=64)
    a = LlamaConfig.from_dict(dict(base, rope_theta=500000.0, rope_scaling=scaling))
    b = LlamaConfig.from_dict(dict(base, rope_parameters=dict(scaling, rope_theta=500000.0)))
    c = LlamaConfig.from_dict(dict(base, rope_theta=500000.0, rope_scaling=dict(scaling, type="llama3")))
    assert a.rope_scaling == b.rope_scaling == c.rope_scaling and a.rope_theta == b.rope_theta == 500000.0


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_rope_table_matches_plain_formula(name):
    raw = rc.TINY_CONFIGS[name]
    params = dict(LlamaConfig.from_dict(raw).to_model_spec().layers[0].mixer.params["position"].params)
    assert params.pop("name") == "model.layers.0.self_attn.rotary_emb"   # where a checkpoint may keep the table
    table = rope_inverse_frequencies(**params)
    want = plain_llama.rope_inv_freq(raw).to(torch.float32)
    assert table.dtype == torch.float32 and torch.allclose(table, want, rtol=1e-6, atol=0)
    if name == "B":  # scaling really changes the low frequencies, keeps the high ones
        plain = rope_inverse_frequencies(params["head_dim"], params["theta"])
        assert torch.equal(table[0], plain[0]) and table[-1] < plain[-1] / 7.9


@pytest.mark.parametrize("patch,match", [
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_type"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "missing"),
    (dict(vocab_size=0), "positive"),
])
def test_refusals(patch, match):
    raw = dict(rc.TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(raw)


def test_missing_key_is_named():
    raw = dict(rc.TINY_A)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_dict(raw)


def test_registry_by_architecture_and_model_type(tmp_path):
    assert "LlamaForCausalLM" in registered_architectures()
    assert model_spec_from_config(rc.TINY_A).architecture == "LlamaForCausalLM"
    by_type = {k: v for k, v in rc.TINY_A.items() if k != "architectures"}
    assert model_spec_from_config(by_type).architecture == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="unsupported architecture"):
        model_spec_from_config(dict(rc.TINY_A, architectures=["Nope"], model_type="nope"))
    (tmp_path / "config.json").write_text(json.dumps(rc.TINY_B))
    assert model_spec_from_folder(tmp_path).vocab_size == rc.TINY_B["vocab_size"]
    with pytest.raises(FileNotFoundError):
        model_spec_from_folder(tmp_path / "absent")


def test_register_another_architecture():
    def factory(raw):
        return LlamaConfig.from_dict(raw).to_model_spec()

    register_architecture("ToyForCausalLM", factory, model_types=("toy",))
    try:
        assert model_spec_from_config(dict(rc.TINY_A, architectures=["ToyForCausalLM"])).vocab_size == 256
        with pytest.raises(ValueError):
            register_architecture("ToyForCausalLM", factory)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_schedule_is_validated():
    spec = LlamaConfig.from_dict(rc.TINY_A).to_model_spec()
    fields = {f: getattr(spec, f) for f in spec.__dataclass_fields__}
    ModelSpec(**dict(fields, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))))
    with pytest.raises(ValueError, match="names layer"):
        ModelSpec(**dict(fields, schedule=(ScheduleEntry(5),)))
    with pytest.raises(ValueError, match="earlier entry"):
        ModelSpec(**dict(fields, schedule=(ScheduleEntry(0, cache_of=0),)))
    with pytest.raises(ValueError, match="borrows"):
        ModelSpec(**dict(fields, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(1, cache_of=1))))


def test_engine_config_validation():
    cfg = KVCoreConfig(model_config=ModelConfig(model="x", dtype="bf16"))
    assert cfg.model_config.dtype == "bfloat16" and cfg.cache_config.block_size == 16
    assert ModelConfig(model="x", dtype="fp32").dtype == "float32"
    for bad in (lambda: ModelConfig(model="x", dtype="int8"), lambda: ModelConfig(model="x", max_model_len=0),
                lambda: CacheConfig(block_size=0), lambda: CacheConfig(gpu_memory_utilization=1.5),
                lambda: SchedulerConfig(max_num_seqs=0), lambda: SchedulerConfig(long_prefill_token_threshold=-1)):
        with pytest.raises(ValueError):
            bad()
    assert PartSpec("x", {"a": 1}).with_params(b=2).params == {"a": 1, "b": 2}


def test_sampling_options_are_validated_and_named():
    from kvcore_b200 import SamplingParams

    params = SamplingParams.from_mapping(dict(max_tokens=3, temperature=0.0, top_k=5))
    assert params.greedy and params.kept_logits(100) == 5 and params.kept_logits(3) == 3
    assert not SamplingParams(max_tokens=1).greedy and SamplingParams(max_tokens=1).kept_logits(7) == 7
    for bad, match in ((dict(max_tokens=0), "max_tokens must be positive"),
                       (dict(max_tokens=1, temperature=-0.1), "temperature must be non-negative"),
                       (dict(max_tokens=1, top_p=0.0), "top_p must be in"),
                       (dict(max_tokens=1, top_p=1.5), "top_p must be in"),
                       (dict(max_tokens=1, top_k=0), "top_k must be positive when set"),
                       (dict(max_tokens=1, beam_width=4), "unknown sampling option.*beam_width")):
        with pytest.raises(ValueError, match=match):
            SamplingParams.from_mapping(bad)


def test_generation_requests_are_taken_in_either_form():
    from kvcore_b200 import GenerationRequest, SamplingParams

    given = GenerationRequest("a", SamplingParams(max_tokens=2), prompt_token_ids=(1, 2))
    assert GenerationRequest.coerce(given) is given
    made = GenerationRequest.coerce(dict(request_id=7, sampling_params=dict(max_tokens=2), prompt_token_ids=[3, 4]))
    assert made.request_id == "7" and made.prompt_token_ids == (3, 4) and made.sampling_params.max_tokens == 2
    chat = GenerationRequest.coerce(dict(request_id="c", sampling_params=SamplingParams(max_tokens=1),
                                         messages=[{"role": "user", "content": "hi"}]))
    assert chat.prompt_token_ids is None and chat.messages[0]["content"] == "hi"


def test_debug_fill_of_freed_pages_is_validated():
    from kvcore_b200 import CacheConfig

    assert CacheConfig(debug_fill_freed_pages="poison").debug_fill_freed_pages == "poison"
    with pytest.raises(ValueError, match="debug_fill_freed_pages"):
        CacheConfig(debug_fill_freed_pages="nan")
    with pytest.raises(ValueError, match="prefix"):
        CacheConfig(debug_fill_freed_pages="zero", enable_prefix_caching=True)
