"""Weights: safetensors round trip, binding by name with packing, the collected error, dtypes,
and the seeded random-weights mode."""
from __future__ import annotations

import json

import pytest
import torch

from kvcore_b200.config import model_spec_from_config
from kvcore_b200.parts import build_model
from kvcore_b200.weights import (
    SafetensorsError, SafetensorsFile, WeightLoadError, load_model_weights, load_state_dict,
    random_state_dict, write_random_model, write_safetensors,
)

import plain_llama
import replay_cases as rc


def _model(name, dtype=torch.float32):
    return build_model(model_spec_from_config(rc.TINY_CONFIGS[name]), dtype=dtype, device="cpu")


def test_safetensors_round_trip_agrees_with_the_safetensors_package(tmp_path):
    tensors = {
        "a.weight": torch.randn(3, 5).to(torch.bfloat16),
        "b": torch.randn(7),
        "table": torch.arange(12, dtype=torch.int32).view(3, 4),
        "empty": torch.empty(0, 4),
    }
    path = tmp_path / "x.safetensors"
    write_safetensors(path, tensors, metadata={"k": "v"})
    with SafetensorsFile(path) as handle:
        assert sorted(handle.names()) == sorted(tensors) and handle.metadata == {"k": "v"}
        for name, tensor in tensors.items():
            assert handle.tensor(name).dtype == tensor.dtype and torch.equal(handle.tensor(name), tensor)
    theirs = plain_llama.load_weights(tmp_path)
    for name, tensor in tensors.items():
        assert torch.equal(theirs[name], tensor)


def test_safetensors_refuses_garbage(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x10\x00\x00\x00\x00\x00\x00\x00not json at all!")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)
    path.write_bytes(b"\xff" * 8 + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_load_binds_by_name_and_packs(name, tmp_path):
    config = rc.TINY_CONFIGS[name]
    folder = write_random_model(tmp_path / "m", config, 5, dtype="float32")
    assert json.loads((folder / "config.json").read_text())["vocab_size"] == config["vocab_size"]
    model = _model(name)
    loaded = load_model_weights(model, folder)
    theirs = plain_llama.load_weights(folder)
    assert loaded == set(theirs)
    block = model.blocks[1]
    p = "model.layers.1"
    q, k, v = (theirs[f"{p}.self_attn.{x}_proj.weight"] for x in "qkv")
    assert torch.equal(block.mixer.qkv_weight, torch.cat((q, k, v)))
    gate, up = theirs[f"{p}.mlp.gate_proj.weight"], theirs[f"{p}.mlp.up_proj.weight"]
    group = block.feed_forward.group
    assert group == (8 if config["intermediate_size"] % 8 == 0 else 0)
    if group:   # gate and up rows alternate in runs of 8
        packed = torch.stack((gate.view(-1, group, gate.shape[1]), up.view(-1, group, up.shape[1])), dim=1)
        assert torch.equal(block.feed_forward.gate_up_weight, packed.reshape(-1, gate.shape[1]))
    else:
        assert torch.equal(block.feed_forward.gate_up_weight, torch.cat((gate, up)))
    assert torch.equal(block.feed_forward.down_weight, theirs[f"{p}.mlp.down_proj.weight"])
    assert torch.equal(model.final_norm.weight, theirs["model.norm.weight"])
    if config["tie_word_embeddings"]:
        assert model.lm_head.weight is model.embedding.weight and "lm_head.weight" not in theirs
    else:
        assert torch.equal(model.lm_head.weight, theirs["lm_head.weight"])
    if config.get("attention_bias"):
        assert torch.equal(block.mixer.qkv_bias[: q.shape[0]], theirs[f"{p}.self_attn.q_proj.bias"])
        assert float(block.mixer.qkv_bias.abs().sum()) > 0


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    tensors = random_state_dict(rc.TINY_A, 0, dtype="float32")
    del tensors["model.norm.weight"]
    del tensors["model.layers.0.mlp.up_proj.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # ignorable
    tensors["model.extra.weight"] = torch.zeros(3)
    tensors["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(5, 64)
    with pytest.raises(WeightLoadError) as info:
        load_state_dict(_model("A"), tensors)
    err = info.value
    assert err.missing == ["model.layers.0.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.extra.weight"]
    assert err.wrong_shape == [("model.layers.1.self_attn.k_proj.weight", (5, 64), (32, 64))]
    text = str(err)
    for needle in ("missing", "unexpected", "wrong shapes", "model.norm.weight", "model.extra.weight", "[5, 64]"):
        assert needle in text
    load_state_dict(_model("A"), tensors, strict=False)  # non-strict loads what matches


def test_tied_head_in_checkpoint_is_ignored():
    tensors = random_state_dict(rc.TINY_B, 1, dtype="float32")
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    load_state_dict(_model("B"), tensors)


def test_precision_policy():
    """bf16 stays bf16; a bf16 checkpoint upcasts exactly into a float32 model; a norm weight the
    file stores in 32-bit stays 32-bit in a bf16 model; integer tables become int32."""
    tensors = random_state_dict(rc.TINY_A, 0, dtype="bfloat16")
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    model = _model("A", torch.bfloat16)
    tensors["model.norm.weight"] = torch.full((64,), 1.00001, dtype=torch.float32)
    load_state_dict(model, tensors)
    assert model.blocks[0].mixer.qkv_weight.dtype == torch.bfloat16
    assert model.final_norm.weight.dtype == torch.float32 and float(model.final_norm.weight[0]) == pytest.approx(1.00001)
    assert model.blocks[0].mixer_norm.weight.dtype == torch.bfloat16
    wide = _model("A", torch.float32)
    load_state_dict(wide, tensors)
    assert torch.equal(wide.embedding.weight, tensors["model.embed_tokens.weight"].float())
    from kvcore_b200.parts.base import WeightSlot
    from kvcore_b200.weights import load_named_tensors

    table = torch.zeros(4, dtype=torch.int32)
    load_named_tensors([WeightSlot("t", table)], [("t", torch.tensor([1, 2, 3, 4], dtype=torch.int64))])
    assert table.tolist() == [1, 2, 3, 4] and table.dtype == torch.int32


def test_random_weights_are_seeded():
    a = random_state_dict(rc.TINY_A, 0, dtype="float32")
    b = random_state_dict(rc.TINY_A, 0, dtype="float32")
    c = random_state_dict(rc.TINY_A, 1, dtype="float32")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert torch.equal(a["model.norm.weight"], torch.ones(64))
    assert 0.015 < float(a["model.embed_tokens.weight"].std()) < 0.025
    half = random_state_dict(rc.TINY_A, 0, dtype="bfloat16")
    assert torch.equal(half["lm_head.weight"], a["lm_head.weight"].to(torch.bfloat16))


def test_missing_folder_and_files(tmp_path):
    with pytest.raises(FileNotFoundError):
        load_model_weights(_model("A"), tmp_path / "nope")
    (tmp_path / "config.json").write_text("{}")
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model_weights(_model("A"), tmp_path)


def test_sharded_checkpoint_with_index(tmp_path):
    tensors = random_state_dict(rc.TINY_A, 0, dtype="float32")
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    model = _model("A")
    assert load_model_weights(model, tmp_path) == set(names)
