"""The command line as a user runs it: ``bin/kvcore_offline_batch`` in a process of its own, on a
written model folder, requests from ``--prompt-tokens-file``.  Behaviour to match: the reference's
offline-batch script builds a config from its options, hands all requests to ``LLMEngine.generate``
and prints run metadata, one section per request with its token ids, and a timing summary
(scripts/run_llm_engine_offline_batch.py:177-231)."""
from __future__ import annotations

import ast
import json
import re
import subprocess
import sys

import numpy as np
import pytest

import plain_llama
import replay_cases as rc

pytestmark = pytest.mark.gpu


def run_cli(*args, timeout=300):
    command = [sys.executable, str(rc.ROOT / "bin" / "kvcore_offline_batch"), *map(str, args)]
    return subprocess.run(command, capture_output=True, text=True, timeout=timeout)


def parse_outputs(stdout: str) -> dict[str, tuple[str, list[int]]]:
    found = {}
    for match in re.finditer(r"^\[(?P<id>[^\]]+)\] finish_reason=(?P<reason>\S+)\ntoken_ids=(?P<ids>\(.*\))$", stdout, re.M):
        found[match["id"]] = (match["reason"], list(ast.literal_eval(match["ids"])))
    return found


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_offline_batch_program_generates_the_plain_tokens(dtype, tmp_path):
    config = rc.TINY_CONFIGS["D"]
    folder = rc.write_model(tmp_path / "model", config, 3, "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompts = {f"req-{i}": rc.random_tokens(config["vocab_size"], n, seed)
               for i, (n, seed) in enumerate(((70, 24), (150, 7), (33, 10)))}
    specs = [dict(request_id=rid, prompt_token_ids=tokens) for rid, tokens in prompts.items()]
    specs[2]["sampling_params"] = dict(max_tokens=5)
    (tmp_path / "requests.json").write_text(json.dumps(specs))
    log = tmp_path / "logs" / "run.log"
    result = run_cli("--model", folder, "--dtype", dtype, "--prompt-tokens-file", tmp_path / "requests.json",
                     "--max-tokens", 8, "--block-size", 16, "--num-gpu-blocks", 64, "--max-model-len", 256,
                     "--max-num-seqs", 4, "--max-num-scheduled-tokens", 96, "--max-num-partial-prefills", 4,
                     "--max-long-partial-prefills", 4, "--attn-backend", "triton_paged", "--log-level", "WARNING",
                     "--log-file", log)
    assert result.returncode == 0, result.stderr[-2000:]
    out = result.stdout
    for section in ("=== Run Metadata ===", "=== Offline Requests ===", "=== Detokenized Outputs ===", "=== Timing Summary ==="):
        assert section in out
    assert "num_requests=3" in out and "output_tokens=21" in out and re.search(r"generate_sec=\d+\.\d+", out)
    assert log.read_text() == out
    outputs = parse_outputs(out)
    assert list(outputs) == list(prompts)
    for rid, prompt in prompts.items():
        reason, tokens = outputs[rid]
        steps = 5 if rid == "req-2" else 8
        assert reason == "length" and len(tokens) == steps
        if dtype == "float32":
            assert tokens == plain_llama.greedy_generate(config, weights, prompt, steps)
        else:   # a near-tie may fall either way: every token is one the plain logits put next to the largest
            logits = plain_llama.forward_logits(config, weights, prompt + tokens).numpy()
            bound = 2 * 2e-2 * np.abs(logits).max()
            for index, token in enumerate(tokens):
                row = logits[len(prompt) + index - 1]
                assert row[token] >= row.max() - bound


def test_offline_batch_program_with_random_weights_and_seeded_sampling(tmp_path):
    """No weight file at all (``--random-weights``), seeded random prompts, temperature sampling with a
    seed: two runs print the same tokens."""
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(rc.TINY_CONFIGS["A"]))
    runs = []
    for _ in range(2):
        result = run_cli("--model", folder, "--random-weights", "--seed", 3, "--random-prompts", "3:21", "--max-tokens", 6,
                         "--temperature", 0.8, "--top-k", 50, "--top-p", 0.9, "--sample-seed", 11, "--num-gpu-blocks", 32,
                         "--max-model-len", 128, "--log-level", "ERROR")
        assert result.returncode == 0, result.stderr[-2000:]
        outputs = parse_outputs(result.stdout)
        assert len(outputs) == 3 and all(len(tokens) == 6 for _, tokens in outputs.values())
        runs.append(outputs)
    assert runs[0] == runs[1]


def test_offline_batch_program_fails_loudly_on_a_bad_folder(tmp_path):
    result = run_cli("--model", tmp_path / "nothing-here", "--num-gpu-blocks", 8)
    assert result.returncode != 0 and "config.json" in result.stderr
