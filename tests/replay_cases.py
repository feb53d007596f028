"""Builders of replay traces (the four cuttings) and helpers to run them and collect logits.

A trace is a list of steps in the replay program's input format.  Every builder asks for
logits at every position of every request, so that any two cuttings of the same requests
can be compared position by position, and each against the plain implementation.
"""
from __future__ import annotations

import json
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

TINY_A = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=256, hidden_size=64,
    intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    max_position_embeddings=128, tie_word_embeddings=False, rms_norm_eps=1e-5, rope_theta=10000.0,
    hidden_act="silu",
)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=515, hidden_size=96,
    intermediate_size=160, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
    head_dim=32, max_position_embeddings=256, tie_word_embeddings=True, rms_norm_eps=1e-6,
    rope_theta=500000.0, hidden_act="silu", attention_bias=True, mlp_bias=True,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
)
# the baseline's second configuration exactly as stated: vocabulary 512, no biases, pages of 8 tokens
# (TINY_B above is its superset with an odd vocabulary and biases on every projection)
TINY_B_AS_STATED = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=512, hidden_size=96,
    intermediate_size=160, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
    head_dim=32, max_position_embeddings=256, tie_word_embeddings=True, rms_norm_eps=1e-6,
    rope_theta=500000.0, hidden_act="silu",
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
)
# a third shape: head size 48 (a step of 16, no power of two), 6 heads in 3 groups, odd widths
TINY_C = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=301, hidden_size=120,
    intermediate_size=200, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, max_position_embeddings=512, tie_word_embeddings=False, rms_norm_eps=3e-6,
    rope_theta=250000.0, hidden_act="silu", logit_scale=0.5,
    rope_parameters=dict(rope_type="linear", rope_theta=250000.0, factor=2.0),
)
# head size 128 (the serving kernels' fast paths: TMA decode, tcgen05 prefill), 2 q heads a kv head
TINY_D = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=384, hidden_size=192,
    intermediate_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=128, max_position_embeddings=1024, tie_word_embeddings=False, rms_norm_eps=1e-5,
    rope_theta=500000.0, hidden_act="silu",
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=128),
)
# head size 64, 3 q heads a kv head
TINY_E = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=200, hidden_size=160,
    intermediate_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2,
    head_dim=64, max_position_embeddings=1024, tie_word_embeddings=True, rms_norm_eps=1e-6,
    rope_theta=10000.0, hidden_act="silu",
)
TINY_CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "B8": TINY_B_AS_STATED}
TINY_SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "B8": 1}
# tokens a cache page holds in the replay tests of each configuration
TINY_PAGE_SIZES = {"A": 16, "B": 16, "C": 16, "D": 16, "E": 16, "B8": 8}


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


# ---- traces --------------------------------------------------------------------------------------
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one step each."""
    steps = []
    for index, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": index, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}],
                      "end": [rid]})
    return steps


def trace_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}],
                      "end": []})
        for pos in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[pos]], "want": [0]}],
                          "end": [rid] if pos == len(tokens) - 1 else []})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def cut(tokens: list[int], sizes: list[int]) -> list[list[int]]:
    """Portions of changing size (cycled), never shorter than one token."""
    out, cursor, index = [], 0, 0
    while cursor < len(tokens):
        size = sizes[index % len(sizes)]
        out.append(tokens[cursor : cursor + size])
        cursor += size
        index += 1
    return out


def trace_chunks(requests: dict[str, list[int]], sizes=(7, 3, 16, 2, 5, 1, 9, 2)) -> list[dict]:
    steps = []
    for rid, tokens in requests.items():
        portions = cut(tokens, list(sizes))
        for index, portion in enumerate(portions):
            steps.append({"step": len(steps),
                          "entries": [{"id": rid, "tokens": portion, "want": list(range(len(portion)))}],
                          "end": [rid] if index == len(portions) - 1 else []})
    return steps


def trace_mixed(requests: dict[str, list[int]], max_live: int = 4, seed: int = 0,
                prompt_fraction: float = 0.6) -> list[dict]:
    """Up to ``max_live`` requests at a time: the first part of each goes in portions of
    changing size, the rest token by token, portions of some beside decode tokens of
    others; a request sometimes sits a step out.  New requests start as old ones end."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: dict[str, dict] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, tokens = waiting.pop(0)
            live[rid] = {"tokens": tokens, "done": 0, "prompt": max(1, int(len(tokens) * prompt_fraction))}
        entries, ended = [], []
        for rid, state in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2 and entries:
                continue  # sits this step out
            remaining_prompt = state["prompt"] - state["done"]
            if remaining_prompt > 0:
                size = int(min(remaining_prompt, rng.choice([2, 3, 5, 8, 13, 21])))
            else:
                size = 1
            portion = state["tokens"][state["done"] : state["done"] + size]
            entries.append({"id": rid, "tokens": portion, "want": list(range(len(portion)))})
            state["done"] += len(portion)
            if state["done"] >= len(state["tokens"]):
                ended.append(rid)
                del live[rid]
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def peak_tokens(steps: list[dict], page: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of ``page``."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-n // page) * page for n in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


def keep_wants(steps: list[dict], keep: dict[str, set[int]]) -> list[dict]:
    """The same steps asking for logits only at the positions (counted within each request) that
    ``keep`` names: for models whose vocabulary makes logits at every position too much to write."""
    seen: dict[str, int] = {}
    out = []
    for step in steps:
        entries = []
        for entry in step["entries"]:
            base = seen.get(entry["id"], 0)
            wanted = [w for w in entry["want"] if base + w in keep.get(entry["id"], ())]
            entries.append(dict(entry, want=wanted))
            seen[entry["id"]] = base + len(entry["tokens"])
        for rid in step["end"]:
            seen.pop(rid, None)
        out.append(dict(step, entries=entries))
    return out


# ---- running --------------------------------------------------------------------------------------
def collect(steps: list[dict], out_dir: Path, vocab: int) -> dict[tuple[str, int], np.ndarray]:
    """Map (request id, position in the request) -> logits row, from the written files."""
    seen: dict[str, int] = {}
    rows: dict[tuple[str, int], np.ndarray] = {}
    for step in steps:
        wanted = [(e["id"], seen.get(e["id"], 0) + w) for e in step["entries"] for w in e["want"]]
        path = out_dir / f"{step['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
            for key, row in zip(wanted, data):
                rows[key] = row
        else:
            assert not path.exists()
        for e in step["entries"]:
            seen[e["id"]] = seen.get(e["id"], 0) + len(e["tokens"])
        for rid in step["end"]:
            seen.pop(rid, None)
    return rows


def run_inprocess(model_dir, dtype: str, steps: list[dict], out_dir: Path, max_tokens: int,
                  device: str = "cuda:0", page_size: int = 16, fill_freed_pages: str | None = None):
    from kvcore_b200.engine.trace_replay import build_replay, replay_stream

    step_function, kv = build_replay(str(model_dir), dtype, max_tokens, page_size=page_size, device=device,
                                     fill_freed_pages=fill_freed_pages)
    lines = [json.dumps(step) for step in steps]
    done: list[str] = []
    replay_stream(step_function, kv, lines, Path(out_dir), done.append)
    assert done == [f"done {step['step']}" for step in steps]
    kv.check_invariants()
    assert not kv.live_requests()
    return step_function, kv


def run_on(step_function, kv, steps: list[dict], out_dir: Path) -> None:
    """Replay ``steps`` on a step function that is there already (a large model is loaded once)."""
    from kvcore_b200.engine.trace_replay import replay_stream

    done: list[str] = []
    replay_stream(step_function, kv, [json.dumps(step) for step in steps], Path(out_dir), done.append)
    assert done == [f"done {step['step']}" for step in steps]
    kv.check_invariants()
    assert not kv.live_requests()


def run_subprocess(model_dir, dtype: str, steps: list[dict], out_dir: Path, max_tokens: int, env=None):
    """Drive bin/trace_run as a user would: write a step, wait for its ``done`` line, go on."""
    cmd = [str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    process = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
                               env=env or os.environ.copy())
    try:
        for step in steps:
            process.stdin.write(json.dumps(step) + "\n")
            process.stdin.flush()
            line = process.stdout.readline().strip()
            assert line == f"done {step['step']}", f"expected 'done {step['step']}', got {line!r}"
        process.stdin.close()
        assert process.wait(timeout=120) == 0
    finally:
        if process.poll() is None:
            process.kill()


def write_model(folder, config: dict, seed: int, dtype: str = "bfloat16"):
    from kvcore_b200.weights import write_random_model

    return write_random_model(folder, config, seed, 0.02, dtype)
