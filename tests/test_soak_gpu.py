"""Randomised runs of the whole engine on the tiny configuration with the serving head size (128, so the
streaming products, the TMA decode attention and the tcgen05 prompt attention are the kernels at work):
requests of random lengths, some with a common beginning, through ``LLMEngine`` with few pages (waiting,
preemption and recomputation), small token budgets (prompts in portions beside decoded tokens), every page
size, with and without reuse of prefix pages, with and without freed pages overwritten.  In float32 the
tokens must be the plain implementation's greedy ones; in bfloat16 every token must be one that the plain
32-bit logits put within the rounding bound of the largest."""
from __future__ import annotations

import random

import numpy as np
import pytest

import plain_llama
import replay_cases as rc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_through_the_engine(seed, tmp_path):
    from kvcore_b200 import CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SamplingParams, SchedulerConfig
    from kvcore_b200.engine.llm_engine import LLMEngine
    import kvcore_b200.kernels as K

    config = rc.TINY_CONFIGS["D"]
    vocab = config["vocab_size"]
    folder = rc.write_model(tmp_path / "m", config, 3, "bfloat16")
    weights = plain_llama.load_weights(folder)
    rng = random.Random(500 + seed)
    count = rng.randint(6, 12)
    shared = rc.random_tokens(vocab, rng.randint(20, 90), 900 + seed)
    prompts = []
    for i in range(count):
        body = rc.random_tokens(vocab, rng.choice([1, 2, 5, 17, 33, 64, rng.randint(1, 200)]), 1000 * seed + i)
        prompts.append((shared + body) if rng.random() < 0.4 else body)
    steps = [rng.randint(1, 20) for _ in range(count)]
    block = rng.choice([8, 16, 32])
    longest = max(len(p) + s for p, s in zip(prompts, steps))
    pages = -(-longest // block) + rng.randint(2, 8)          # room for the longest request and little more
    budget = rng.choice([8, 24, 64, 200])
    prefix = rng.random() < 0.5
    fill = None if prefix else rng.choice([None, "poison"])
    expected = [plain_llama.greedy_generate(config, weights, p, s) for p, s in zip(prompts, steps)]
    for dtype in ("float32", "bfloat16"):
        engine = LLMEngine(KVCoreConfig(
            model_config=ModelConfig(model=str(folder), dtype=dtype, max_model_len=-(-longest // block) * block),
            cache_config=CacheConfig(block_size=block, num_gpu_blocks=pages, enable_prefix_caching=prefix,
                                     debug_fill_freed_pages=fill),
            scheduler_config=SchedulerConfig(max_num_seqs=rng.choice([2, 4, 8]), max_num_scheduled_tokens=budget,
                                             max_num_partial_prefills=4, max_long_partial_prefills=4),
            device_config=DeviceConfig(device="cuda:0")))
        outputs = engine.generate([
            dict(request_id=f"r{i}", prompt_token_ids=p, sampling_params=SamplingParams(max_tokens=s, temperature=0.0))
            for i, (p, s) in enumerate(zip(prompts, steps))])
        got = [list(o.output_token_ids) for o in outputs]
        what = f"seed {seed} {dtype}: block {block}, {pages} pages, budget {budget}, prefix reuse {prefix}, fill {fill}"
        if dtype == "float32":
            assert got == expected, what
        else:
            for prompt, tokens in zip(prompts, got):
                logits = plain_llama.forward_logits(config, weights, prompt + tokens).numpy()
                bound = 4e-2 * np.abs(logits).max()
                for index, token in enumerate(tokens):
                    row = logits[len(prompt) + index - 1]
                    assert row[token] >= row.max() - bound, f"{what}: token {index} of {tokens}"
        assert K.read_status() == 0, what
        engine.engine_core.model_runner.kv_manager.check_invariants()
