"""The plain implementation against the reference's own model code: tests/golden/ holds logits
that Baizx98/KVCore's Llama3ForCausalLM produced on three tiny random models (made by
tests/golden/make_golden.py): the baseline's two configurations and one with biases, full multi-head
attention and a logit scale.  Also checks the plain implementation against itself: float64,
and the sampling masks."""
from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

import plain_llama
from golden.make_golden import state_dict_hash
from kvcore_b200.weights import SafetensorsFile, random_state_dict

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def golden():
    record = json.loads((GOLDEN / "reference_logits.json").read_text())
    return record, SafetensorsFile(GOLDEN / "reference_logits.safetensors")


@pytest.mark.parametrize("name", ["A", "B", "BIAS"])
def test_plain_matches_reference_model_code(golden, name):
    record, logits = golden
    config = record["configs"][name]
    weights = random_state_dict(config, record["seeds"][name], 0.02, "float32")
    # the golden file holds logits, not weights: they are drawn again from the seed, and if this torch
    # draws other numbers than the one that made the file, the anchor is gone and must be made again
    assert state_dict_hash(weights) == record["weights_sha256"][name], (
        f"torch {torch.__version__} draws other random weights than torch {record['torch']}, which made the golden "
        "file: run tests/golden/make_golden.py against a checkout of the reference again")
    if name == "BIAS":
        assert any(key.endswith("q_proj.bias") for key in weights) and any(key.endswith("down_proj.bias") for key in weights)
        assert config["logit_scale"] != 1.0
    for index, tokens in enumerate(record["tokens"][name]):
        want = logits.tensor(f"{name}/seq{index}")
        got = plain_llama.forward_logits(config, weights, tokens)
        assert got.shape == want.shape
        torch.testing.assert_close(got, want, rtol=0, atol=2e-6)


def test_plain_float64_and_bf16_rounding_bracket_float32():
    record = json.loads((GOLDEN / "reference_logits.json").read_text())
    config = record["configs"]["B"]
    weights = random_state_dict(config, 1, 0.02, "float32")
    tokens = record["tokens"]["B"][2]
    f32 = plain_llama.forward_logits(config, weights, tokens)
    f64 = plain_llama.forward_logits(config, weights, tokens, compute=torch.float64)
    bf16 = plain_llama.forward_logits(config, weights, tokens, round_to=torch.bfloat16)
    scale = float(f64.abs().max())
    assert float((f32.double() - f64).abs().max()) < 2e-6 * scale
    err = float((bf16 - f32).abs().max()) / scale
    assert 1e-4 < err < 1e-2  # what a faithful bfloat16 run loses; the bf16 GPU tests allow 1.2e-2 on the tiny models


def test_window_changes_only_far_positions():
    record = json.loads((GOLDEN / "reference_logits.json").read_text())
    config = record["configs"]["A"]
    weights = random_state_dict(config, 0, 0.02, "float32")
    tokens = record["tokens"]["A"][1]
    full = plain_llama.forward_logits(config, weights, tokens)
    windowed = plain_llama.forward_logits(config, weights, tokens, window=5)
    assert torch.equal(full[:5], windowed[:5]) and not torch.allclose(full[8:], windowed[8:], atol=1e-6)


def test_sampling_masks():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 3.0])
    kept = plain_llama.masked_logits(logits, 1.0, 2, 1.0)
    assert torch.isfinite(kept).tolist() == [True, False, False, False, True]
    kept = plain_llama.masked_logits(logits, 1.0, None, 0.5)
    assert torch.isfinite(kept).tolist() == [False, False, False, False, True]
    kept = plain_llama.masked_logits(logits, 1.0, None, 0.9)
    assert torch.isfinite(kept).tolist() == [True, True, False, False, True]
    assert torch.equal(plain_llama.masked_logits(logits, 2.0, None, 1.0), logits / 2.0)
